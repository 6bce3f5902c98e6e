"""The legacy out-variant operators hpu::cast_to_fp8 and hpu::fp8_gemm (pre-allocated out / amax;
hpu_ops/backend/fp8_ops.cpp:123-166,312-366), with the cases, value ranges and tolerances of the
reference's own tests (tests/pytest_working/lazy/test_hpu_fp8_ops.py:34-132) plus bit-exactness
against the oracle, which the v2 operators share their kernels with."""
import numpy as np
import pytest
import torch

from oracle import hpu_oracle as O

pytestmark = pytest.mark.gpu
FP8 = [torch.float8_e5m2, torch.float8_e4m3fn]
# tests/pytest_working/fp8_utils.py:53-55
REF_FP8_MAX = {torch.float8_e5m2: 57344 * 0.9, torch.float8_e4m3fn: 240 * 0.9}


@pytest.fixture(autouse=True)
def _status():
    import b200_hpu_ops
    yield
    assert b200_hpu_ops.device_status() == 0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("stochastic", [True, False])
@pytest.mark.parametrize("out_dtype", FP8)
def test_cast_to_fp8_out_variant(dtype, stochastic, out_dtype):
    shape, scale_v = (4, 8), 1.6
    g = torch.Generator().manual_seed(3)
    pos = torch.rand(shape, generator=g).to(dtype) * 30 + 10
    x = torch.cat((pos, -pos))
    scale = torch.tensor(scale_v, dtype=torch.float32)
    scale_inv = scale.reciprocal()
    want8, want_amax = O.cast_to_fp8_v2(x, scale, False, True, out_dtype)
    unscaled = O.cast_from_fp8(want8, scale_inv, dtype)

    casted = torch.empty((shape[0] * 2, shape[1]), dtype=out_dtype, device="cuda")
    amax = torch.empty((), dtype=torch.float32, device="cuda")
    r = torch.ops.hpu.cast_to_fp8(x.cuda(), scale.cuda(), stochastic, casted, amax)
    assert r[0].data_ptr() == casted.data_ptr() and r[1].data_ptr() == amax.data_ptr()  # written in place
    back = torch.ops.hpu.cast_from_fp8(casted, scale_inv.cuda(), dtype).cpu()
    if stochastic:
        assert torch.allclose(back.float(), unscaled.float(), rtol=0.26, atol=0.0)
    else:
        assert torch.equal(casted.cpu().view(torch.uint8), want8.view(torch.uint8))
        assert torch.equal(back, unscaled)
    assert amax.cpu() == x.abs().max().float() == want_amax


def test_cast_to_fp8_out_variant_checks():
    x = torch.ones(4, 8, device="cuda")
    amax = torch.empty((), device="cuda")
    with pytest.raises(RuntimeError, match="same shape"):
        torch.ops.hpu.cast_to_fp8(x, None, False, torch.empty(4, 4, dtype=torch.float8_e4m3fn, device="cuda"), amax)
    with pytest.raises(RuntimeError, match="float or bfloat16"):
        torch.ops.hpu.cast_to_fp8(x.to(torch.float16), None, False, torch.empty(4, 8, dtype=torch.float8_e4m3fn, device="cuda"), amax)


@pytest.mark.parametrize("shapeA, shapeB", [((2, 3, 4, 2), (2, 3, 4, 8)), ((64, 48), (64, 112))])
@pytest.mark.parametrize("bias", [True, False])
@pytest.mark.parametrize("accumulate", [True, False])
@pytest.mark.parametrize("scaleA, scaleB", [(True, True), (True, False), (False, True), (False, False)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("fp8_dtype", FP8)
def test_fp8_gemm_out_variant(shapeA, shapeB, bias, accumulate, scaleA, scaleB, dtype, fp8_dtype):
    g = torch.Generator().manual_seed(11)
    A = torch.rand(shapeA, generator=g).to(dtype) * 10 + 30.0
    B = torch.rand(shapeB, generator=g).to(dtype) * 10 + 30.0
    sA = (REF_FP8_MAX[fp8_dtype] / A.abs().max().float()) if scaleA else None
    sB = (REF_FP8_MAX[fp8_dtype] / B.abs().max().float()) if scaleB else None
    sAi = None if sA is None else sA.reciprocal()
    sBi = None if sB is None else sB.reciprocal()
    out_shape = shapeA[:-2] + (shapeA[-1],) + (shapeB[-1],)
    bias_t = (torch.rand(out_shape, generator=g).to(dtype) * 10 + 30.0) if bias else None
    out = torch.full(out_shape, 1000.0, dtype=dtype)
    out_d = out.cuda()
    cu = lambda t: None if t is None else t.cuda()  # noqa: E731

    A8, _ = torch.ops.hpu.cast_to_fp8_v2(A.cuda(), cu(sA), False, False, fp8_dtype)
    B8, _ = torch.ops.hpu.cast_to_fp8_v2(B.cuda(), cu(sB), False, False, fp8_dtype)
    r = torch.ops.hpu.fp8_gemm(A8, True, B8, False, out_d, dtype, cu(sAi), cu(sBi), cu(bias_t), accumulate, out_d)
    assert r.data_ptr() == out_d.data_ptr()

    # the reference's own bound: integer-truncated percentage error against the unquantised product
    ref = torch.matmul(A.transpose(-2, -1).float(), B.float())
    if bias:
        ref = ref + bias_t.float()
    if accumulate:
        ref = ref + out.float()
    pct = torch.abs(((out_d.cpu().float() - ref) / ref) * 100).to(torch.int)
    assert np.amax(pct.numpy()) <= 15
    # and ours: the oracle on the same fp8 operands
    want = O.fp8_gemm_v2(A8.cpu(), True, B8.cpu(), False, out, dtype, sAi, sBi, bias_t, accumulate, None)
    assert O.rel_frobenius(out_d, want) <= 1e-2
