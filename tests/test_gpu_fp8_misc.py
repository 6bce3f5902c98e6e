"""softmax_fp8, sum_fp8 and in_place_interleave_ on the GPU against the oracle; cases mirror
tests/pytest_working/any_mode/test_hpu_fp8_ops_any_mode.py:795-824,980-1048 and
test_hpu_sum_fp8.py:30-55 of the reference."""
import pytest
import torch

from oracle import hpu_oracle as O

E4M3, E5M2 = torch.float8_e4m3fn, torch.float8_e5m2


@pytest.fixture(scope="module")
def ops():
    import b200_hpu_ops
    assert torch.cuda.is_available()
    return b200_hpu_ops


def _fp8_steps_apart(a8, b8):
    """|difference| in fp8 codes (same format, same sign region)."""
    a, b = a8.view(torch.uint8).int(), b8.view(torch.uint8).int()
    return (a - b).abs()


# ---------------------------------------------------------------- softmax_fp8
@pytest.mark.gpu
@pytest.mark.parametrize("is_scale,input_dtype", [(True, E4M3), (True, torch.bfloat16), (False, torch.bfloat16)])
@pytest.mark.parametrize("is_inv_attn_heads", [True, False])
@pytest.mark.parametrize("fused_add_shape", [None, (5, 4, 4, 6), (5, 1, 1, 6)])
def test_softmax_fp8_reference_cases(ops, is_scale, is_inv_attn_heads, fused_add_shape, input_dtype):
    g = torch.Generator().manual_seed(17)
    shape = (5, 4, 4, 6)
    x = (torch.rand(shape, generator=g) * 4.0).to(torch.bfloat16)
    xin = x.to(input_dtype)
    s_in = torch.tensor(0.05) if is_scale else None
    s_out = torch.tensor(2.5) if is_scale else None
    heads = torch.tensor(0.1) if is_inv_attn_heads else None
    fa = torch.rand(fused_add_shape, generator=g).to(torch.bfloat16) if (fused_add_shape and is_scale) else None
    cu = lambda t: None if t is None else t.cuda()  # noqa: E731
    got = torch.ops.hpu.softmax_fp8(xin.cuda(), -1, cu(s_in), cu(s_out), cu(heads), cu(fa)).cpu()
    want = O.softmax_fp8(xin, -1, s_in, s_out, heads, fa)
    assert got.dtype == want.dtype == (E4M3 if is_scale else torch.bfloat16)
    if is_scale:
        d = _fp8_steps_apart(got, want)
        assert int(d.max()) <= 1 and float((d != 0).float().mean()) < 0.02
    else:
        assert torch.allclose(got.float(), want.float(), rtol=2 ** -7, atol=1e-6)
    # the reference test's own emulation and tolerance (bf16 arithmetic step by step)
    ref = x.to(input_dtype).to(torch.bfloat16)
    if is_inv_attn_heads:
        ref = ref * heads
    if is_scale:
        ref = ref * s_in
        if fa is not None:
            ref = ref + fa
    ref = torch.softmax(ref, -1).to(torch.bfloat16)
    if is_scale:
        ref = (ref * s_out).to(E4M3)
    assert torch.allclose(got.float(), ref.float(), atol=1e-2, rtol=0.1251)
    # scalar overloads give the same bytes
    if is_scale:
        if fa is None or True:
            g2 = torch.ops.hpu.softmax_fp8.Scalar_scales(xin.cuda(), -1, 0.05, 2.5, cu(heads), cu(fa)).cpu()
            assert torch.equal(g2.view(torch.uint8), got.view(torch.uint8))
        if is_inv_attn_heads:
            g3 = torch.ops.hpu.softmax_fp8.Scalar(xin.cuda(), -1, 0.05, 2.5, 0.1, cu(fa)).cpu()
            d3 = _fp8_steps_apart(g3, got)  # host product of the two scalars vs device products
            assert int(d3.max()) <= 1


@pytest.mark.gpu
@pytest.mark.parametrize("dim", [0, 1, -2])
def test_softmax_fp8_over_another_dimension(ops, dim):
    """The reference hands any `dim` to its kernel (softmax_fp8_gen.cpp:65-160); here the row kernel
    runs on the tensor with `dim` moved to the end."""
    g = torch.Generator().manual_seed(9 + dim)
    x = (torch.randn(6, 40, 24, generator=g) * 2).to(torch.bfloat16)
    r = torch.ops.hpu.softmax_fp8(x.cuda(), dim)
    e = O.softmax_fp8(x, dim)
    assert r.shape == e.shape and r.dtype == torch.bfloat16
    assert torch.allclose(r.cpu().float(), e.float(), atol=4e-3, rtol=2e-2)
    r8 = torch.ops.hpu.softmax_fp8(x.cuda(), dim, 0.5, 240.0)
    e8 = O.softmax_fp8(x, dim, 0.5, 240.0)
    assert r8.dtype == torch.float8_e4m3fn
    d = (r8.cpu().view(torch.uint8).int() - e8.view(torch.uint8).int()).abs()
    assert int(d.max()) <= 1 and float((d > 0).float().mean()) < 0.02


@pytest.mark.gpu
@pytest.mark.parametrize("cols", [24, 256, 1000, 4096, 6144, 8192, 12288, 16384])
def test_softmax_fp8_row_kernel_branches(ops, cols):
    """The register-resident row kernel's special paths (one warp per row up to 4096 elements, two up
    to 8192, four up to 16384): a negative input scale (the packed maximum runs on sign-flipped inputs), an output scale that is a power of two (folded into the
    normalisation), rows with -inf entries, and rows that are NaN as a whole (a NaN, a +inf, or
    only -inf in the row)."""
    g = torch.Generator().manual_seed(cols)
    x = (torch.randn(12, cols, generator=g) * 3).to(torch.bfloat16)
    x[1, ::3] = float("-inf")
    x[2, 5] = float("nan")
    x[3, 7] = float("inf")
    x[4, :] = float("-inf")
    for s_in, s_out in [(-0.5, 240.0), (0.25, 256.0), (-1.0, 0.5), (1.0, 1.0)]:
        got = torch.ops.hpu.softmax_fp8(x.cuda(), -1, s_in, s_out).cpu()
        want = O.softmax_fp8(x, -1, s_in, s_out)
        gn, wn = got.float().isnan(), want.float().isnan()
        assert torch.equal(gn, wn), (s_in, s_out, gn.sum(), wn.sum())
        assert bool(gn[2].all()) and bool(gn[4].all()) and not bool(gn[0].any())
        ok = ~gn
        d = (got.view(torch.uint8).int() - want.view(torch.uint8).int()).abs()[ok]
        assert int(d.max()) <= 1 and float((d > 0).float().mean()) < 0.02, (s_in, s_out)
    gb = torch.ops.hpu.softmax_fp8(x.cuda(), -1).cpu()  # bf16 output, no scales
    wb = O.softmax_fp8(x, -1)
    assert torch.equal(gb.isnan(), wb.isnan())
    assert torch.allclose(gb.float().nan_to_num(0.0), wb.float().nan_to_num(0.0), rtol=2 ** -7, atol=1e-6)


@pytest.mark.gpu
@pytest.mark.parametrize("cols", [64, 1000, 4096, 8192])
def test_softmax_fp8_e4m3_input_rows(ops, cols):
    """e4m3 scores in, e4m3 probabilities out (the reference's is_scale / float8 input case) through
    the register-resident row kernel: the input is exact in bf16, so the result is the bf16 kernel's."""
    g = torch.Generator().manual_seed(cols + 1)
    x = (torch.randn(9, cols, generator=g) * 3).to(E4M3)
    x.view(torch.uint8)[2, 5] = 0x7F  # a NaN score: the whole row is NaN
    for s_in, s_out in [(0.5, 240.0), (-0.25, 256.0)]:
        got = torch.ops.hpu.softmax_fp8(x.cuda(), -1, s_in, s_out).cpu()
        want = O.softmax_fp8(x, -1, s_in, s_out)
        gn, wn = got.float().isnan(), want.float().isnan()
        assert torch.equal(gn, wn) and bool(gn[2].all())
        d = (got.view(torch.uint8).int() - want.view(torch.uint8).int()).abs()[~gn]
        assert int(d.max()) <= 1 and float((d > 0).float().mean()) < 0.02
        same = torch.ops.hpu.softmax_fp8(x.to(torch.bfloat16).cuda(), -1, s_in, s_out).cpu()
        assert torch.equal(same.view(torch.uint8), got.view(torch.uint8))


@pytest.mark.gpu
@pytest.mark.parametrize("cols", [2048, 8192])
def test_softmax_fp8_fused_add_long_rows(ops, cols):
    """fused_add (an attention-mask shaped addend, broadcast over the head dimension) with rows held by
    one and by two warps."""
    g = torch.Generator().manual_seed(cols)
    x = (torch.randn(2, 3, 4, cols, generator=g) * 2).to(torch.bfloat16)
    fa = (torch.randn(2, 1, 4, cols, generator=g)).to(torch.bfloat16)
    got = torch.ops.hpu.softmax_fp8(x.cuda(), -1, torch.tensor(0.5).cuda(), torch.tensor(200.0).cuda(), None, fa.cuda()).cpu()
    want = O.softmax_fp8(x, -1, torch.tensor(0.5), torch.tensor(200.0), None, fa)
    d = _fp8_steps_apart(got, want)
    assert int(d.max()) <= 1 and float((d != 0).float().mean()) < 0.02


@pytest.mark.gpu
def test_softmax_fp8_long_rows_and_errors(ops):
    g = torch.Generator().manual_seed(3)
    x = (torch.randn(37, 4099, generator=g) * 3).to(torch.bfloat16)
    got = torch.ops.hpu.softmax_fp8(x.cuda(), 1, None, None, None, None).cpu()
    want = O.softmax_fp8(x, 1)
    assert torch.allclose(got.float(), want.float(), rtol=2 ** -7, atol=1e-7)
    assert torch.allclose(got.float().sum(-1), torch.ones(37), atol=2e-2)
    s = torch.tensor(1.0).cuda()
    with pytest.raises(RuntimeError, match="Output and input scales must be both given or None"):
        torch.ops.hpu.softmax_fp8(x.cuda(), -1, s, None, None, None)
    with pytest.raises(RuntimeError, match="then input scale must be given"):
        torch.ops.hpu.softmax_fp8(x.cuda().to(E4M3), -1, None, None, None, None)
    with pytest.raises(RuntimeError, match="FusedAdd available only for Float8 output"):
        torch.ops.hpu.softmax_fp8(x.cuda(), -1, None, None, None, x.cuda())
    with pytest.raises(RuntimeError, match="must be of torch.bfloat16 or torch.float8_e4m3fn"):
        torch.ops.hpu.softmax_fp8(x.cuda().float(), -1, None, None, None, None)
    assert ops.device_status() == 0


# ---------------------------------------------------------------- sum_fp8
@pytest.mark.gpu
@pytest.mark.parametrize("dim", [0, 1, 2, (0, 1), (0, 2), None])
@pytest.mark.parametrize("keep_dim", [True, False])
@pytest.mark.parametrize("dtype", [E5M2, E4M3])
@pytest.mark.parametrize("out_dtype", [None, torch.float])
def test_sum_fp8_reference_cases(ops, dim, keep_dim, dtype, out_dtype):
    g = torch.Generator().manual_seed(29)
    x = (torch.randn((10, 20, 30), generator=g) * 10.0).to(dtype)
    d = None if dim is None else ([dim] if isinstance(dim, int) else list(dim))
    got = torch.ops.hpu.sum_fp8(x.cuda(), d, keep_dim, out_dtype).cpu()
    exact = torch.sum(x.to(torch.float64), d if d is not None else list(range(3)), keep_dim)
    assert got.shape == exact.shape
    if out_dtype:
        assert got.dtype == out_dtype
        # fp32 accumulation in a fixed order: within a few ulp of the exact sum
        assert torch.allclose(got.double(), exact, rtol=4e-7, atol=4e-7 * float(x.float().abs().sum() / max(1, exact.numel())))
    else:
        assert got.dtype == dtype
        want = O.sum_fp8(x, d, keep_dim, None)
        steps = _fp8_steps_apart(got, want)
        assert int(steps.max()) <= 1 and float((steps != 0).float().mean()) <= 0.02


@pytest.mark.gpu
def test_sum_fp8_large_and_deterministic(ops):
    g = torch.Generator(device="cuda").manual_seed(1)
    x = torch.randn(3, 1 << 20, device="cuda", generator=g).to(E4M3)
    a = torch.ops.hpu.sum_fp8(x, [1], False, torch.float)
    b = torch.ops.hpu.sum_fp8(x, [1], False, torch.float)
    assert torch.equal(a, b)
    exact = x.double().sum(1)
    assert torch.allclose(a.double(), exact, rtol=1e-5, atol=1e-2)
    tot = torch.ops.hpu.sum_fp8(x, None, False, torch.float)
    assert tot.shape == () and abs(float(tot) - float(exact.sum())) < 0.05
    col = torch.ops.hpu.sum_fp8(x, [0], True, torch.float)
    assert col.shape == (1, 1 << 20) and torch.allclose(col.double(), x.double().sum(0, keepdim=True), atol=1e-5)
    assert ops.device_status() == 0


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [E4M3, E5M2])
@pytest.mark.parametrize("shape,dim", [((4100, 512), 0), ((3, 700, 48), 1), ((2, 4097, 16), 1), ((5000, 40), 0)])
def test_sum_fp8_over_an_outer_dimension(ops, dtype, shape, dim):
    """Sums over a dimension that is not the last: positions of the kept inner dimensions in groups of
    16 per thread when their number is a multiple of 16 (else one per thread), the reduce range in
    chunks; fp32 accumulation, the same bits on every run."""
    g = torch.Generator(device="cuda").manual_seed(shape[0])
    x = (torch.randn(shape, device="cuda", generator=g) * 4).to(dtype)
    a = torch.ops.hpu.sum_fp8(x, [dim], False, torch.float)
    b = torch.ops.hpu.sum_fp8(x, [dim], False, torch.float)
    assert torch.equal(a, b)
    exact = x.double().sum(dim)
    assert a.shape == exact.shape
    assert torch.allclose(a.double(), exact, rtol=1e-5, atol=1e-3 * float(x.float().abs().max()))
    assert ops.device_status() == 0


# ---------------------------------------------------------------- in_place_interleave_
@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.bfloat16, E5M2, E4M3, torch.float32])
@pytest.mark.parametrize("shape", [(8, 2, 2, 5), (4, 1, 1, 1), (64, 3, 5, 7), (1024, 2, 4, 8), (8, 4, 512, 136), (16, 1, 1, 48),
                                   (12, 3, 1, 37), (20, 1, 40, 1000)])
def test_in_place_interleave(ops, dtype, shape):
    g = torch.Generator().manual_seed(shape[0])
    x = (torch.randn(shape, generator=g) * 10.0).to(torch.bfloat16).to(dtype)
    xc = x.cuda()
    r = torch.ops.hpu.in_place_interleave_(xc)
    assert r.data_ptr() == xc.data_ptr()
    want = O.in_place_interleave(x.view(torch.uint8) if dtype in (E5M2, E4M3) else x)
    got = xc.cpu().view(torch.uint8) if dtype in (E5M2, E4M3) else xc.cpu()
    assert torch.equal(got, want)


@pytest.mark.gpu
def test_in_place_interleave_errors(ops):
    with pytest.raises(RuntimeError, match="Input has to be a 4D tensor."):
        torch.ops.hpu.in_place_interleave_(torch.zeros(8, 2, 2, device="cuda"))
    with pytest.raises(RuntimeError, match="Batch size has to be a multiple of 4."):
        torch.ops.hpu.in_place_interleave_(torch.zeros(6, 2, 2, 2, device="cuda"))


# ---------------------------------------------------------------- conv2d_fp8
@pytest.mark.gpu
@pytest.mark.parametrize("scaleA", [True, False])
@pytest.mark.parametrize("scaleB", [True, False])
@pytest.mark.parametrize("bias", [True, False])
@pytest.mark.parametrize("out_dtype", [torch.float, torch.bfloat16])
@pytest.mark.parametrize("fp8_dtype", [E5M2, E4M3])
def test_conv2d_fp8_reference_case(ops, scaleA, scaleB, bias, out_dtype, fp8_dtype):
    """test_hpu_fp8_ops_any_mode.py:830-897: N,C,H,W = 8,3,28,28, 16 output channels, 2x2 kernel."""
    g = torch.Generator().manual_seed(41)
    x = torch.rand((8, 3, 28, 28), generator=g).to(out_dtype).to(fp8_dtype)
    w = torch.rand((16, 3, 2, 2), generator=g).to(out_dtype).to(fp8_dtype)
    b = torch.rand(16, generator=g).to(out_dtype).to(fp8_dtype).to(out_dtype) if bias else None
    sa = torch.tensor(1.4).to(out_dtype) if scaleA else None
    sb = torch.tensor(2.3).to(out_dtype) if scaleB else None
    cu = lambda t: None if t is None else t.cuda()  # noqa: E731
    args = [x.cuda(), w.cuda(), cu(b), (1, 1), (0, 0), (1,), 1, out_dtype]
    if sa is not None or sb is not None:
        args += [cu(sa), cu(sb)]
    got = torch.ops.hpu.conv2d_fp8(*args).cpu()
    want = O.conv2d_fp8(x, w, b, (1, 1), (0, 0), (1, 1), 1, out_dtype, sa, sb)
    assert got.shape == want.shape == (8, 16, 27, 27) and got.dtype == out_dtype
    assert O.rel_frobenius(got, want) <= (1e-2 if out_dtype == torch.bfloat16 else 1e-5)
    # the reference test's own bound
    ref = torch.nn.functional.conv2d(x.to(out_dtype), w.to(out_dtype), None, (1, 1), (0, 0), (1, 1), 1)
    ref = ref * ((sa if sa is not None else 1) * (sb if sb is not None else 1))
    if b is not None:
        ref = ref + b.reshape(1, -1, 1, 1)
    rtol = 0.02 if (out_dtype == torch.bfloat16 and (scaleA or scaleB)) else 1e-2
    assert torch.allclose(got.float(), ref.float(), atol=1e-2, rtol=rtol)


@pytest.mark.gpu
@pytest.mark.parametrize("cfg", [
    dict(N=2, C=32, H=17, W=19, Co=48, k=(3, 3), stride=(2, 1), padding=(1, 2), dilation=(1, 2), groups=1),
    dict(N=3, C=16, H=9, W=9, Co=24, k=(3, 1), stride=(1, 1), padding=(0, 0), dilation=(1, 1), groups=4),
    dict(N=1, C=64, H=14, W=14, Co=128, k=(1, 1), stride=(1, 1), padding=(0, 0), dilation=(1, 1), groups=1),
    # 512 channels x 3 rows x 66 bytes do not fit one block's shared memory: two channel chunks per output line
    dict(N=1, C=520, H=6, W=64, Co=16, k=(3, 3), stride=(1, 1), padding=(1, 1), dilation=(1, 1), groups=1),
    # channel groups of whole 16-byte pieces take the channels-last path (transposed copy, 16-byte gather, columns
    # ordered window-first): many channels, groups of 16 and 48 channels, a partial 64-channel tile, odd image sizes
    dict(N=1, C=512, H=6, W=64, Co=16, k=(3, 3), stride=(1, 1), padding=(1, 1), dilation=(1, 1), groups=1),
    dict(N=2, C=64, H=13, W=7, Co=32, k=(3, 2), stride=(2, 1), padding=(1, 1), dilation=(1, 2), groups=4),
    dict(N=3, C=96, H=5, W=5, Co=6, k=(5, 5), stride=(1, 1), padding=(2, 2), dilation=(1, 1), groups=2),
    dict(N=1, C=80, H=31, W=33, Co=40, k=(1, 3), stride=(3, 2), padding=(0, 1), dilation=(1, 1), groups=1),
    dict(N=2, C=6, H=11, W=23, Co=8, k=(2, 3), stride=(1, 2), padding=(1, 0), dilation=(2, 1), groups=2),
    # image rows too wide for the patch kernel's shared memory (3 channels x 3 lines x 12 KB): the fallback kernel
    dict(N=1, C=3, H=4, W=12288, Co=8, k=(3, 3), stride=(1, 1), padding=(1, 1), dilation=(1, 1), groups=1),
])
def test_conv2d_fp8_shapes_and_scalar_overload(ops, cfg):
    g = torch.Generator().manual_seed(cfg["C"])
    x = torch.randn((cfg["N"], cfg["C"], cfg["H"], cfg["W"]), generator=g).to(E4M3)
    w = (torch.randn((cfg["Co"], cfg["C"] // cfg["groups"]) + cfg["k"], generator=g) * 0.3).to(E4M3)
    b = torch.randn(cfg["Co"], generator=g)
    got = torch.ops.hpu.conv2d_fp8.scalar(x.cuda(), w.cuda(), b.cuda(), cfg["stride"], cfg["padding"], cfg["dilation"], cfg["groups"],
                                          torch.float, 0.5, 0.25).cpu()
    want = O.conv2d_fp8(x, w, b, cfg["stride"], cfg["padding"], cfg["dilation"], cfg["groups"], torch.float, 0.5, 0.25)
    assert got.shape == want.shape
    assert O.rel_frobenius(got, want) <= 1e-5
    with pytest.raises(RuntimeError, match="Input and weight must be 4D tensors"):
        torch.ops.hpu.conv2d_fp8(x.cuda()[0], w.cuda())
    with pytest.raises(RuntimeError, match="Bias must be 1D tensor with size equal to weight dim0"):
        torch.ops.hpu.conv2d_fp8(x.cuda(), w.cuda(), b.cuda()[:-1])
    with pytest.raises(RuntimeError, match="Multi-element scale tensors are not supported yet."):
        torch.ops.hpu.conv2d_fp8(x.cuda(), w.cuda(), None, (1, 1), (0, 0), (1, 1), cfg["groups"], None, torch.ones(2).cuda(), None)
    assert ops.device_status() == 0
