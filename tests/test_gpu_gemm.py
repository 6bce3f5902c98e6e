"""fp8_gemm_v2 on the GPU against the CPU oracle (fp32 accumulation).  Tolerance: relative
Frobenius error <= 1e-2 for deterministic rounding; the reference's own cases
(tests/pytest_working/any_mode/test_hpu_fp8_ops_any_mode.py:352-703) keep their tolerances."""
import os

import numpy as np
import pytest
import torch

from conftest import GOLDEN
from oracle import hpu_oracle as O

pytestmark = pytest.mark.gpu
FP8 = [torch.float8_e5m2, torch.float8_e4m3fn]
TOL = 1e-2
_DT = {"torch.float32": torch.float32, "torch.bfloat16": torch.bfloat16,
       "torch.float8_e5m2": torch.float8_e5m2, "torch.float8_e4m3fn": torch.float8_e4m3fn}


@pytest.fixture(scope="module")
def ops():
    import b200_hpu_ops
    return b200_hpu_ops


@pytest.fixture(autouse=True)
def _no_device_timeouts(ops):
    yield
    assert ops.device_status() == 0, "a bounded wait inside a kernel ran out"


def _rand_fp8(shape, fp8, g, lo=-2.0, hi=2.0):
    return (torch.rand(shape, generator=g) * (hi - lo) + lo).to(fp8)


def _cuda(x):
    return None if x is None else (x.cuda() if isinstance(x, torch.Tensor) else x)


def _check(A, tA, B, tB, D, od, sA=None, sB=None, bias=None, acc=False, shape=None, tol=TOL):
    r = torch.ops.hpu.fp8_gemm_v2(_cuda(A), tA, _cuda(B), tB, _cuda(D), od, _cuda(sA), _cuda(sB), _cuda(bias), acc, shape)
    e = O.fp8_gemm_v2(A, tA, B, tB, D, od, sA, sB, bias, acc, shape)
    assert r.dtype == od and list(r.shape) == list(e.shape)
    err = O.rel_frobenius(r, e)
    assert err <= tol, err
    return r


def test_reference_golden_cases(ops):
    z = np.load(os.path.join(GOLDEN, "gemm_small.npz"))
    for i in range(int(z["n"])):
        k = f"g{i}"
        dtype, fp8 = _DT[z[k + "_meta"][0]], _DT[z[k + "_meta"][1]]
        A = torch.from_numpy(z[k + "_A"]).to(dtype)
        B = torch.from_numpy(z[k + "_B"]).to(dtype)
        bias = torch.from_numpy(z[k + "_bias"]).to(dtype)
        sA, sB = torch.from_numpy(z[k + "_sA"]), torch.from_numpy(z[k + "_sB"])
        ref = torch.from_numpy(z[k + "_ref"])
        A8, _ = torch.ops.hpu.cast_to_fp8_v2(A.cuda(), sA.cuda(), False, False, fp8)
        B8, _ = torch.ops.hpu.cast_to_fp8_v2(B.cuda(), sB.cuda(), False, False, fp8)
        D = torch.full(ref.shape, 1000.0, dtype=dtype)
        for use_bias in (False, True):
            for acc in (False, True):
                r = torch.ops.hpu.fp8_gemm_v2(A8, True, B8, False, D.cuda(), dtype, sA.reciprocal().cuda(),
                                              sB.reciprocal().cuda(), bias.cuda() if use_bias else None, acc)
                e = ref + (bias.float() if use_bias else 0) + (D.float() if acc else 0)
                pd = torch.abs(((r.cpu().float() - e) / e) * 100).to(torch.int)
                assert int(pd.max()) <= 15
                o = O.fp8_gemm_v2(A8.cpu(), True, B8.cpu(), False, D, dtype, sA.reciprocal(), sB.reciprocal(),
                                  bias if use_bias else None, acc)
                assert O.rel_frobenius(r, o) <= TOL


@pytest.mark.parametrize("tA", [False, True])
@pytest.mark.parametrize("tB", [False, True])
@pytest.mark.parametrize("fa,fb", [(FP8[0], FP8[0]), (FP8[1], FP8[1]), (FP8[0], FP8[1])])
@pytest.mark.parametrize("M,N,K", [(24, 36, 12), (130, 257, 96), (128, 256, 128), (64, 48, 200)])
def test_transposes_and_odd_sizes(ops, tA, tB, fa, fb, M, N, K):
    g = torch.Generator().manual_seed(M + N + K)
    A = _rand_fp8((K, M) if tA else (M, K), fa, g)
    B = _rand_fp8((N, K) if tB else (K, N), fb, g)
    bias = torch.randn(N, generator=g).to(torch.bfloat16)
    sB = torch.rand(N, generator=g) + 0.5
    D = torch.randn(M, N, generator=g)
    for od in (torch.bfloat16, torch.float32):
        _check(A, tA, B, tB, None, od)
        _check(A, tA, B, tB, D, od, torch.tensor(0.25), sB, bias, True, [1, N])


@pytest.mark.parametrize("shapeA,shapeB", [((2, 1, 4, 2), (1, 3, 4, 8)), ((2, 1, 4, 2), (4, 8)), ((4, 2), (3, 4, 8))])
def test_batched_broadcast_shapes(ops, shapeA, shapeB):
    # test_hpu_fp8_ops_any_mode.py:504-514 (trans_A = True)
    g = torch.Generator().manual_seed(1)
    A = _rand_fp8(shapeA, torch.float8_e5m2, g)
    B = _rand_fp8(shapeB, torch.float8_e5m2, g)
    r = _check(A, True, B, False, None, torch.float32, torch.tensor(0.5), torch.tensor(2.0))
    bias = torch.randn(r.shape, generator=g)
    _check(A, True, B, False, bias, torch.bfloat16, None, None, bias, True)


@pytest.mark.parametrize("shape_a,shape_b", [((10,), (10,)), ((2, 10), (10,)), ((10,), (10, 2)), ((4, 8, 16), (16,)),
                                             ((8,), (2, 4, 8, 16))])
@pytest.mark.parametrize("tA", [True, False])
@pytest.mark.parametrize("tB", [True, False])
def test_1d_operands(ops, shape_a, shape_b, tA, tB):
    # test_hpu_fp8_ops_any_mode.py:534-596
    if (tA and len(shape_a) == 1) or (tB and len(shape_b) == 1):
        pytest.skip("Configuration not supported")
    g = torch.Generator().manual_seed(2)
    A = _rand_fp8(shape_a, torch.float8_e5m2, g, 30, 40)
    B = _rand_fp8(shape_b, torch.float8_e5m2, g, 30, 40)
    A_in = A.transpose(-2, -1).contiguous() if tA else A
    B_in = B.transpose(-2, -1).contiguous() if tB else B
    sA, sB = torch.tensor(3.14, dtype=torch.bfloat16), torch.tensor(0.75, dtype=torch.bfloat16)
    r = torch.ops.hpu.fp8_gemm_v2(A_in.cuda(), tA, B_in.cuda(), tB, None, torch.bfloat16, sA.cuda(), sB.cuda(), None,
                                  False)
    ref = torch.matmul(A.to(torch.bfloat16), B.to(torch.bfloat16)) * torch.mul(sA, sB)
    assert list(r.shape) == list(ref.shape)
    pd = torch.abs(((r.cpu().float() - ref.float()) / ref.float()) * 100).to(torch.int)
    assert int(pd.max()) <= 15
    assert O.rel_frobenius(r, O.fp8_gemm_v2(A_in, tA, B_in, tB, None, torch.bfloat16, sA, sB)) <= TOL


@pytest.mark.parametrize("axis", [0, 1])
def test_scale_shape_lists(ops, axis):
    # test_hpu_fp8_ops_any_mode.py:599-657: per-column (axis 0) / per-row (axis 1) list scales
    g = torch.Generator().manual_seed(3)
    A = _rand_fp8((12, 24), torch.float8_e4m3fn, g, 30, 40)
    B = _rand_fp8((24, 36), torch.float8_e4m3fn, g, 30, 40)
    n = 12 if axis == 1 else 36
    sa = [float(torch.rand(1, generator=g) * 100)]
    sb = (torch.rand(n, generator=g) * 100).tolist()
    shape = [n, 1] if axis == 1 else [1, n]
    r = torch.ops.hpu.fp8_gemm_v2(A.cuda(), False, B.cuda(), False, None, torch.bfloat16, sa, sb, None, False, shape)
    ref = torch.matmul(A.to(torch.bfloat16), B.to(torch.bfloat16)) * (torch.tensor(sa) * torch.tensor(sb).reshape(shape))
    np.testing.assert_allclose(r.cpu().float().numpy(), ref.float().numpy(), atol=1e-3, rtol=1e-2)
    with pytest.raises(RuntimeError, match=r"Number of scale elements \(\d+\) is not equal to number of scale_shape"):
        torch.ops.hpu.fp8_gemm_v2(A.cuda(), False, B.cuda(), False, None, torch.bfloat16, sa, sb, None, False, [1, n + 1])


@pytest.mark.parametrize("scaleA", [16, 14])
@pytest.mark.parametrize("scaleB", [0.00390625, 0.23])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_scalar_overload(ops, scaleA, scaleB, dtype):
    # test_hpu_fp8_ops_any_mode.py:660-703
    g = torch.Generator().manual_seed(4)
    A = _rand_fp8((12, 24), torch.float8_e4m3fn, g, 30, 40)
    B = _rand_fp8((24, 36), torch.float8_e4m3fn, g, 30, 40)
    r = torch.ops.hpu.fp8_gemm_v2(A.cuda(), False, B.cuda(), False, None, dtype, float(scaleA), float(scaleB), None, False)
    ref = torch.matmul(A.to(dtype), B.to(dtype)) * (scaleA * scaleB)
    np.testing.assert_allclose(r.cpu().float().numpy(), ref.float().numpy(), atol=1e-3, rtol=1e-2)
    t = torch.ops.hpu.fp8_gemm_v2(A.cuda(), False, B.cuda(), False, None, dtype, torch.tensor(float(scaleA)).cuda(),
                                  torch.tensor(float(scaleB)).cuda(), None, False)
    assert torch.equal(t, r)  # tensor and scalar overloads agree (…:706-792)


def test_errors(ops):
    f8 = torch.float8_e4m3fn
    A = torch.zeros(4, 8).to(f8).cuda()
    B = torch.zeros(8, 12).to(f8).cuda()
    with pytest.raises(RuntimeError, match="Accumulation tensor must be provided at index 4 for Fp8GemmV2, when "
                                           "accumulate is true"):
        torch.ops.hpu.fp8_gemm_v2(A, False, B, False, None, torch.bfloat16, None, None, None, True)
    with pytest.raises(RuntimeError, match="Common dimension sizes of matmul inputs should be the same. Got 8 and 12"):
        torch.ops.hpu.fp8_gemm_v2(A, False, B, True, None, torch.bfloat16)
    # D is ignored when accumulate is False
    D = torch.full((4, 12), 7.0).cuda()
    r = torch.ops.hpu.fp8_gemm_v2(A, False, B, False, D, torch.bfloat16, None, None, None, False)
    assert float(r.abs().max()) == 0.0


# ---------------------------------------------------------------- the tcgen05 path
def _quantize(x, per_row):
    amax = x.abs().amax(dim=1, keepdim=True) if per_row else x.abs().max()
    scale = 448.0 / amax
    x8, _ = O.cast_to_fp8_v2(x, scale.float(), False, False, torch.float8_e4m3fn, list(scale.shape) if per_row else None)
    return x8, (1.0 / scale).float()


@pytest.mark.parametrize("M,N,K", [(256, 1024, 1024), (128, 256, 128), (384, 512, 256), (200, 300, 144),
                                   (1000, 1112, 4096), (129, 257, 2048)])
def test_tcgen05_projection_shapes(ops, M, N, K):
    """A [M,K] . B [N,K]^T with per-tensor A scale, per-channel B scale and bias (the projection
    form).  Compared both with the oracle and with the generic CUDA kernel (forced through the ABI)."""
    from b200_hpu_ops import abi
    g = torch.Generator().manual_seed(M * 7 + N)
    A8, sa = _quantize(torch.randn(M, K, generator=g).to(torch.bfloat16), False)
    B8, sb = _quantize((torch.randn(N, K, generator=g) * 0.02).to(torch.bfloat16), True)
    bias = (torch.randn(N, generator=g) * 0.01).to(torch.bfloat16)
    r = _check(A8, False, B8, True, None, torch.bfloat16, sa, sb.reshape(-1), bias, False, [1, N])
    slow = abi.fp8_gemm_nt(A8.cuda(), B8.cuda(), torch.bfloat16, float(sa), sb.reshape(-1).cuda(), bias.cuda(),
                           force_generic=True)
    fast = abi.fp8_gemm_nt(A8.cuda(), B8.cuda(), torch.bfloat16, float(sa), sb.reshape(-1).cuda(), bias.cuda())
    assert O.rel_frobenius(fast, slow) <= 2e-3
    assert O.rel_frobenius(fast, r) <= 2e-3
    r32 = _check(A8, False, B8, True, None, torch.float32, sa, sb.reshape(-1), bias, False, [1, N], tol=1e-5)


def test_tcgen05_one_hot_layout_probe(ops):
    """Structured operands make an operand-layout mistake visible as a wrong index rather than
    as noise: A row m is one-hot at k = (7 m) % K, B row n holds n % 13 + k % 5."""
    M, N, K = 256, 512, 512
    A = torch.zeros(M, K)
    A[torch.arange(M), (7 * torch.arange(M)) % K] = 1.0
    B = ((torch.arange(N).reshape(N, 1) % 13) + (torch.arange(K).reshape(1, K) % 5)).float()
    A8, B8 = A.to(torch.float8_e4m3fn), B.to(torch.float8_e4m3fn)
    r = torch.ops.hpu.fp8_gemm_v2(A8.cuda(), False, B8.cuda(), True, None, torch.float32)
    assert torch.equal(r.cpu(), A @ B.t())


@pytest.mark.parametrize("fa,fb", [(FP8[0], FP8[0]), (FP8[0], FP8[1]), (FP8[1], FP8[0])])
def test_tcgen05_mixed_formats_and_epilogue_modes(ops, fa, fb):
    g = torch.Generator().manual_seed(17)
    M, N, K = 256, 384, 512
    A, B = _rand_fp8((M, K), fa, g), _rand_fp8((N, K), fb, g)
    D = torch.randn(M, N, generator=g).to(torch.bfloat16)
    row = torch.rand(M, 1, generator=g) + 0.5
    col = torch.rand(1, N, generator=g) + 0.5
    fullb = torch.randn(M, N, generator=g)
    _check(A, False, B, True, None, torch.bfloat16)
    _check(A, False, B, True, D, torch.bfloat16, row, col, None, True)           # per-row A scale, per-col B scale
    _check(A, False, B, True, D, torch.float32, col, row, fullb, True, [M, 1])   # swapped roles, full bias, fp32 out
    _check(A, False, B, True, None, torch.bfloat16, torch.tensor(0.5), torch.tensor(2.0),
           torch.randn(M, 1, generator=g), False)                                # per-row bias
    _check(A, False, B, True, None, torch.bfloat16, torch.rand(M, N, generator=g), None)  # element-wise scale: generic


@pytest.mark.parametrize("M", [1, 16, 17, 64, 128])
def test_tcgen05_small_m_decode_shapes(ops, M):
    g = torch.Generator().manual_seed(M)
    N, K = 1792, 4096
    A8, sa = _quantize(torch.randn(M, K, generator=g).to(torch.bfloat16), False)
    B8, sb = _quantize((torch.randn(N, K, generator=g) * 0.02).to(torch.bfloat16), True)
    bias = (torch.randn(N, generator=g) * 0.01).to(torch.bfloat16)
    _check(A8, False, B8, True, None, torch.bfloat16, sa, sb.reshape(-1), bias, False, [1, N])
    D = torch.randn(M, N, generator=g)
    _check(A8, False, B8, True, D, torch.float32, torch.rand(M, 1, generator=g) + 0.5, sb.reshape(-1),
           torch.randn(M, N, generator=g), True, [1, N], tol=1e-5)


@pytest.mark.parametrize("M", [1, 5, 8, 9, 16])
@pytest.mark.parametrize("N,K", [(8, 128), (100, 1024), (1000, 2176), (1792, 4096), (264, 6272), (520, 14336)])
def test_few_token_shapes(ops, M, N, K):
    """M <= 16 against K-major weights: the tile kernel with the weights on the lanes, in tiles of
    32..128 weight rows chosen so that the tile count fits the SMs (N < 128 takes the generic
    kernel); N need not be a multiple of the tile height or of 8."""
    g = torch.Generator().manual_seed(M * 7 + N)
    fa, fb = FP8[(M + N) % 2], FP8[(M // 2 + K // 128) % 2]
    A = _rand_fp8((M, K), fa, g)
    B = _rand_fp8((N, K), fb, g, -0.25, 0.25)
    col = torch.rand(N, generator=g) + 0.5
    bias = torch.randn(N, generator=g).to(torch.bfloat16)
    _check(A, False, B, True, None, torch.bfloat16, torch.tensor(0.5), col, bias, False, [1, N])
    D = torch.randn(M, N, generator=g)
    _check(A, False, B, True, D, torch.float32, torch.rand(M, 1, generator=g) + 0.5, col, None, True, [1, N], tol=1e-5)
    # exact small integers: every product and sum is representable, so any misplaced k or row shows
    Ai = ((torch.arange(M).reshape(M, 1) * 3 + torch.arange(K).reshape(1, K)) % 5).float()
    Bi = ((torch.arange(N).reshape(N, 1) % 7) + (torch.arange(K).reshape(1, K) % 3)).float()
    r = torch.ops.hpu.fp8_gemm_v2(Ai.to(FP8[1]).cuda(), False, Bi.to(FP8[1]).cuda(), True, None, torch.float32)
    assert torch.equal(r.cpu(), Ai @ Bi.t())


@pytest.mark.parametrize("M", [1, 16, 128])
def test_decode_shapes_full_width(ops, M):
    """The benchmark's decode shape (14336 weight rows, K = 4096: 104-row tiles) and one whose
    tiles take two rounds (28672 rows)."""
    g = torch.Generator().manual_seed(40 + M)
    for N in (14336, 28672):
        K = 4096 if N == 14336 else 1024
        A = _rand_fp8((M, K), FP8[1], g)
        B = _rand_fp8((N, K), FP8[1], g, -0.25, 0.25)
        col = torch.rand(N, generator=g) + 0.5
        bias = torch.randn(N, generator=g).to(torch.bfloat16)
        _check(A, False, B, True, None, torch.bfloat16, torch.tensor(0.5), col, bias, False, [1, N])


@pytest.mark.parametrize("M,N,K", [(1, 1792, 4096), (16, 14336, 4096), (128, 1024, 1024), (16, 520, 14336)])
def test_static_weights_flag_gives_the_same_bytes(ops, M, N, K):
    """b200q_gemm_args.b_static only changes WHEN the few-token kernel starts to read the weights
    (before or after the kernel in front of it has finished); back-to-back launches with and
    without it, behind a kernel that writes the tokens, give the same bytes."""
    from b200_hpu_ops import abi
    g = torch.Generator(device="cuda").manual_seed(M + N)
    b8 = (torch.randn(N, K, device="cuda", generator=g) * 0.1).to(torch.float8_e4m3fn)
    sb = torch.rand(N, device="cuda", generator=g) + 0.5
    bias = torch.randn(N, device="cuda", generator=g).to(torch.bfloat16)
    outs = []
    for flag in (False, True, True, False):
        a = torch.randn(M, K, device="cuda", generator=torch.Generator(device="cuda").manual_seed(7))
        a8 = a.to(torch.float8_e4m3fn)  # written by the kernel right in front of the GEMM
        outs.append(abi.fp8_gemm_nt(a8, b8, torch.bfloat16, 0.5, sb, bias, b_static=flag))
    torch.cuda.synchronize()
    for o in outs[1:]:
        assert torch.equal(o, outs[0])
    assert ops.device_status() == 0


@pytest.mark.parametrize("N", [516, 520, 518])
@pytest.mark.parametrize("od", [torch.bfloat16, torch.float32])
def test_epilogue_row_segments(ops, N, od):
    """The epilogue's wide loads and stores: accumulate input D and element-wise bias read as 16-byte
    row segments where a row is 16-byte aligned, 8-byte stores when the row pitch is a multiple of 8
    bytes only (N = 516 with bf16), element by element otherwise (N = 518)."""
    g = torch.Generator().manual_seed(N)
    M, K = 300, 256
    A, B = _rand_fp8((M, K), FP8[1], g), _rand_fp8((N, K), FP8[1], g)
    D = torch.randn(M, N, generator=g).to(od)
    fullb = torch.randn(M, N, generator=g).to(od)
    col = torch.rand(1, N, generator=g) + 0.5
    _check(A, False, B, True, D, od, torch.tensor(0.5), col, None, True, [1, N], tol=1e-2 if od == torch.bfloat16 else 1e-5)
    _check(A, False, B, True, D, od, torch.tensor(0.5), col, fullb, True, [1, N], tol=1e-2 if od == torch.bfloat16 else 1e-5)
    _check(A, False, B, True, None, od, torch.tensor(0.5), col, None, False, [1, N], tol=1e-2 if od == torch.bfloat16 else 1e-5)


def test_tcgen05_batch_folds_into_m(ops):
    g = torch.Generator().manual_seed(23)
    A = _rand_fp8((3, 5, 64, 128), torch.float8_e4m3fn, g)
    B = _rand_fp8((256, 128), torch.float8_e4m3fn, g)
    bias = torch.randn(256, generator=g)
    _check(A, False, B, True, None, torch.bfloat16, torch.tensor(0.5), torch.rand(256, generator=g) + 0.5, bias, False, [1, 256])
    _check(A, False, B, True, None, torch.float32, torch.rand(64, 1, generator=g) + 0.5, None, None, False, None, 1e-5)


def test_tcgen05_full_size_properties(ops):
    """M = K = 4096, N = 14336 (the benchmark's GEMM): linearity in A's scale, agreement of a
    sampled set of output rows/columns with the oracle, and equality of two runs."""
    g = torch.Generator(device="cuda").manual_seed(0)
    M, K, N = 4096, 4096, 14336
    A8 = torch.randn(M, K, device="cuda", generator=g).clamp(-3, 3).mul(100).to(torch.float8_e4m3fn)
    B8 = torch.randn(N, K, device="cuda", generator=g).clamp(-3, 3).mul(100).to(torch.float8_e4m3fn)
    sb = torch.rand(N, device="cuda", generator=g) * 1e-4 + 1e-4
    bias = (torch.randn(N, device="cuda", generator=g) * 0.01).to(torch.bfloat16)
    sa = torch.tensor(1e-2, device="cuda")
    r1 = torch.ops.hpu.fp8_gemm_v2(A8, False, B8, True, None, torch.bfloat16, sa, sb, bias, False, [1, N])
    r2 = torch.ops.hpu.fp8_gemm_v2(A8, False, B8, True, None, torch.bfloat16, sa, sb, bias, False, [1, N])
    assert torch.equal(r1, r2)
    rows = torch.tensor([0, 1, 127, 128, 2047, 4095])
    e = O.fp8_gemm_v2(A8[rows].cpu(), False, B8.cpu(), True, None, torch.bfloat16, sa.cpu(), sb.cpu(), bias.cpu(), False, [1, N])
    assert O.rel_frobenius(r1[rows], e) <= TOL
    cols = torch.tensor([0, 255, 256, 7000, 14335])
    e = O.fp8_gemm_v2(A8.cpu(), False, B8[cols].cpu(), True, None, torch.bfloat16, sa.cpu(), sb[cols].cpu(), bias[cols].cpu(),
                      False, [1, len(cols)])
    assert O.rel_frobenius(r1[:, cols], e) <= TOL
    # linearity: doubling the A scale doubles (out - bias)
    r3 = torch.ops.hpu.fp8_gemm_v2(A8, False, B8, True, None, torch.float32, 2 * sa, sb, None, False, [1, N])
    r4 = torch.ops.hpu.fp8_gemm_v2(A8, False, B8, True, None, torch.float32, sa, sb, None, False, [1, N])
    assert torch.equal(r3, 2 * r4)


@pytest.mark.parametrize("tA,tB", [(True, False), (True, True), (False, False)])
@pytest.mark.parametrize("M,N,K", [(384, 512, 320), (208, 1008, 144), (4096, 256, 512), (48, 640, 1024)])
def test_tcgen05_mn_major_operands(ops, tA, tB, M, N, K):
    """Transposed storage orders go to the tensor cores through MN-major descriptors: compare with
    the oracle, with the generic kernel, and exactly on small-integer operands."""
    from b200_hpu_ops import abi
    g = torch.Generator().manual_seed(M + 3 * N + K)
    A = _rand_fp8((K, M) if tA else (M, K), torch.float8_e4m3fn, g)
    B = _rand_fp8((N, K) if tB else (K, N), torch.float8_e5m2, g)
    sB = torch.rand(N, generator=g) + 0.5
    bias = torch.randn(N, generator=g).to(torch.bfloat16)
    _check(A, tA, B, tB, None, torch.bfloat16, torch.tensor(0.5), sB, bias, False, [1, N])
    # exact: small integers, fp32 output, no scales
    Ai = torch.randint(-4, 5, A.shape, generator=g).float()
    Bi = torch.randint(-4, 5, B.shape, generator=g).float()
    r = torch.ops.hpu.fp8_gemm_v2(Ai.to(torch.float8_e4m3fn).cuda(), tA, Bi.to(torch.float8_e4m3fn).cuda(), tB, None,
                                  torch.float32)
    ref = (Ai.t() if tA else Ai) @ (Bi.t() if tB else Bi)
    assert torch.equal(r.cpu(), ref)


def test_tcgen05_mn_major_k_not_multiple_of_16(ops):
    g = torch.Generator().manual_seed(77)
    M, N, K = 256, 384, 200   # both operands MN-major: K needs no alignment
    A = _rand_fp8((K, M), torch.float8_e4m3fn, g)
    B = _rand_fp8((K, N), torch.float8_e4m3fn, g)
    _check(A, True, B, False, None, torch.float32, None, None, None, False, None, tol=1e-5)


@pytest.mark.parametrize("tA,tB", [(False, True), (True, True), (False, False)])
def test_large_k_not_multiple_of_16_is_padded(ops, tA, tB):
    """An operand stored [rows][K] with K % 16 != 0 has no 16-byte row pitch; above 2^26 products the
    operator copies both operands into zero-padded buffers.  Exact on small integers (the zeros add
    nothing), and within tolerance of the oracle with scales, bias and accumulation."""
    g = torch.Generator().manual_seed(5)
    M, N, K = 512, 528, 1000 if not (tA and tB) else 1003
    Ai = torch.randint(-4, 5, (K, M) if tA else (M, K), generator=g).float()
    Bi = torch.randint(-4, 5, (N, K) if tB else (K, N), generator=g).float()
    r = torch.ops.hpu.fp8_gemm_v2(Ai.to(torch.float8_e4m3fn).cuda(), tA, Bi.to(torch.float8_e5m2).cuda(), tB, None,
                                  torch.float32)
    assert torch.equal(r.cpu(), (Ai.t() if tA else Ai) @ (Bi.t() if tB else Bi))
    A = _rand_fp8(tuple(Ai.shape), torch.float8_e4m3fn, g)
    B = _rand_fp8(tuple(Bi.shape), torch.float8_e4m3fn, g)
    D = torch.randn(M, N, generator=g)
    _check(A, tA, B, tB, D, torch.float32, torch.tensor(0.5), torch.rand(N, generator=g) + 0.5,
           torch.randn(N, generator=g), True, [1, N], tol=1e-5)
    # batched, folded into M
    A3 = _rand_fp8((3, 256, 1000), torch.float8_e4m3fn, g)
    B2 = _rand_fp8((528, 1000), torch.float8_e4m3fn, g)
    _check(A3, False, B2, True, None, torch.bfloat16)
    assert ops.device_status() == 0


def test_tcgen05_batched(ops):
    """Batched operands (both with batch dimensions, or a broadcast one) run one tensor-core launch
    per batch item."""
    g = torch.Generator().manual_seed(91)
    A = _rand_fp8((3, 2, 144, 256), torch.float8_e4m3fn, g)
    B = _rand_fp8((3, 1, 320, 256), torch.float8_e4m3fn, g)
    bias = torch.randn(3, 2, 144, 320, generator=g)
    D = torch.randn(3, 2, 144, 320, generator=g)
    _check(A, False, B, True, D, torch.float32, torch.tensor(0.5), torch.rand(320, generator=g) + 0.5, bias, True,
           [1, 320], tol=1e-5)
    Bt = _rand_fp8((2, 256, 320), torch.float8_e5m2, g)   # [K][N] storage, batch broadcast against A's
    _check(A, False, Bt, False, None, torch.bfloat16)


@pytest.mark.parametrize("mid", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("out8", FP8)
@pytest.mark.parametrize("M,N,K", [(256, 512, 256), (16, 384, 512), (130, 257, 96), (24, 36, 12)])
def test_fused_output_cast_equals_unfused_pair(ops, mid, out8, M, N, K):
    """fp8_gemm_cast == cast_to_fp8_v2(fp8_gemm_v2(...), scale) byte for byte (same kernels, the cast
    moved into the epilogue), and close to the oracle's composition."""
    g = torch.Generator().manual_seed(M + N)
    A = _rand_fp8((M, K), torch.float8_e4m3fn, g)
    B = _rand_fp8((N, K), torch.float8_e4m3fn, g)
    sA, sB = torch.tensor(0.5), torch.rand(N, generator=g) + 0.5
    bias = torch.randn(N, generator=g).to(torch.bfloat16)
    scale = 3.7
    fused = torch.ops.b200q.fp8_gemm_cast(A.cuda(), False, B.cuda(), True, None, mid, sA.cuda(), sB.cuda(), bias.cuda(), False,
                                          [1, N], scale, out8)
    plain = torch.ops.hpu.fp8_gemm_v2(A.cuda(), False, B.cuda(), True, None, mid, sA.cuda(), sB.cuda(), bias.cuda(), False, [1, N])
    two, _ = torch.ops.hpu.cast_to_fp8_v2(plain, scale, False, False, out8)
    assert fused.dtype == out8 and fused.shape == (M, N)
    assert torch.equal(fused.view(torch.uint8), two.view(torch.uint8))
    ref, _ = O.cast_to_fp8_v2(O.fp8_gemm_v2(A, False, B, True, None, mid, sA, sB, bias, False, [1, N]), scale, False, False, out8)
    assert O.rel_frobenius(fused.float(), ref.float()) <= 4e-2   # one fp8 step on the few results that sit on a tie


def test_scaled_mm_entry(ops):
    g = torch.Generator().manual_seed(12)
    M, N, K = 64, 256, 128
    a = _rand_fp8((M, K), torch.float8_e4m3fn, g)
    w = _rand_fp8((N, K), torch.float8_e4m3fn, g)
    sa, sw = torch.tensor(0.25), torch.tensor(2.0)
    bias = torch.randn(N, generator=g).to(torch.bfloat16)
    r, _ = torch.ops.b200q.scaled_mm(a.cuda(), w.cuda().t(), sa.cuda(), sw.cuda(), bias.cuda(), None, torch.bfloat16)
    e = O.fp8_gemm_v2(a, False, w, True, None, torch.bfloat16, sa, sw, bias)
    assert O.rel_frobenius(r, e) <= TOL
    r2, _ = torch.ops.b200q.scaled_mm(a.cuda(), w.t().contiguous().cuda(), sa.cuda(), sw.cuda(), None, None, torch.float32)
    assert O.rel_frobenius(r2, O.fp8_gemm_v2(a, False, w, True, None, torch.float32, sa, sw)) <= 1e-5


@pytest.mark.parametrize("out8", FP8)
@pytest.mark.parametrize("M,N,K", [(64, 256, 128), (300, 520, 256), (1, 384, 512), (16, 1792, 1024)])
def test_scaled_mm_fp8_output_and_amax(ops, out8, M, N, K):
    """float8 output of the _scaled_mm-shaped entry: the bytes are cast_to_fp8_v2(bf16 GEMM result,
    scale_result) and the second output is max |out| of the values written
    (hpu_ops/backend/scaled_mm_gen.cpp:283-320), taken inside the GEMM's epilogue."""
    g = torch.Generator().manual_seed(M + N)
    a = _rand_fp8((M, K), torch.float8_e4m3fn, g)
    w = _rand_fp8((N, K), torch.float8_e4m3fn, g)
    sa, sw, sr = torch.tensor(0.25), torch.rand(1, N, generator=g) + 0.5, torch.tensor(0.75)
    bias = torch.randn(N, generator=g).to(torch.bfloat16)
    r8, amax = torch.ops.b200q.scaled_mm(a.cuda(), w.cuda().t(), sa.cuda(), sw.cuda(), bias.cuda(), sr.cuda(), out8)
    assert r8.dtype == out8 and amax.shape == () and amax.dtype == torch.float32
    mid = torch.ops.hpu.fp8_gemm_v2(a.cuda(), False, w.cuda(), True, None, torch.bfloat16, sa.cuda(), sw.reshape(-1).cuda(),
                                    bias.cuda(), False, [1, N])
    two, _ = torch.ops.hpu.cast_to_fp8_v2(mid, sr.cuda(), False, False, out8)
    assert torch.equal(r8.view(torch.uint8), two.view(torch.uint8))
    assert amax.item() == r8.float().abs().max().item()
    # against the oracle: one fp8 step on the few results that sit on a tie of the bf16 intermediate
    ref, _ = O.cast_to_fp8_v2(O.fp8_gemm_v2(a, False, w, True, None, torch.bfloat16, sa, sw.reshape(-1), bias, False, [1, N]),
                              sr, False, False, out8)
    assert O.rel_frobenius(r8.float(), ref.float()) <= 4e-2
