"""convert_from_int4 / convert_from_uint4 on the GPU: bit-exact against the oracle and the golden
vectors made from the reference's own pack / GPTQ helpers
(tests/pytest_working/any_mode/test_hpu_convert_from_int4.py)."""
import os

import numpy as np
import pytest
import torch

from conftest import GOLDEN
from oracle import hpu_oracle as O

pytestmark = pytest.mark.gpu
_DT = {"torch.float32": torch.float32, "torch.bfloat16": torch.bfloat16}


@pytest.fixture(scope="module")
def ops():
    import b200_hpu_ops
    return b200_hpu_ops


def _eq(a, b):
    a, b = a.cpu(), b.cpu()
    return a.dtype == b.dtype and a.shape == b.shape and torch.equal(a.float(), b.float())


def test_golden_unit_and_gptq(ops):
    z = np.load(os.path.join(GOLDEN, "int4.npz"))
    for i in range(int(z["n_unit"])):
        k = f"u{i}"
        variant, zp_kind, od = z[k + "_meta"]
        od = _DT[od]
        packed = torch.from_numpy(z[k + "_packed"]).cuda()
        scale = torch.from_numpy(z[k + "_scale"]).to(od).cuda()
        zp = None
        if zp_kind == "packed":
            zp = torch.from_numpy(z[k + "_zp"]).cuda()
        elif zp_kind == "unpacked":
            zp = torch.from_numpy(z[k + "_zp"]).to(od).cuda()
        fn = torch.ops.hpu.convert_from_int4 if variant == "int4" else torch.ops.hpu.convert_from_uint4
        r = fn(packed, scale, zp, od)
        assert r.dtype == od
        assert torch.equal(r.cpu().float(), torch.from_numpy(z[k + "_ref"])), (k, variant, zp_kind, od)
    for i in range(int(z["n_gptq"])):
        k = f"a{i}"
        od = _DT[z[k + "_meta"][0]]
        is_zp = z[k + "_meta"][1] == "True"
        qw = torch.from_numpy(z[k + "_qweight"]).cuda()
        qz = torch.from_numpy(z[k + "_qzeros"]).cuda()
        sc = torch.from_numpy(z[k + "_scale"]).to(od).cuda()
        ref = torch.from_numpy(z[k + "_ref"])
        r = torch.ops.hpu.convert_from_uint4(qw, sc, qz if is_zp else None, od)
        assert torch.equal(r.cpu().float(), ref), (k, list(z[k + "_meta"]))


@pytest.mark.parametrize("od", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("signed", [True, False])
@pytest.mark.parametrize("shape,group", [((10,), None), ((4, 6, 4), None), ((256, 64), 32), ((3, 64, 24), 16),
                                         ((130, 7), None), ((1024, 512), 128)])
def test_against_oracle(ops, od, signed, shape, group):
    g = torch.Generator().manual_seed(hash((shape, signed)) % 1000)
    real = list(shape)
    real[-1] *= 8
    q = torch.randint(0, 16, real, generator=g)
    packed = O.pack_nibbles(q)
    if group is None:
        sshape = real
    else:
        sshape = real[:-2] + [real[-2] // group, real[-1]]
    scale = (torch.rand(sshape, generator=g) * 0.015 + 0.005).to(od)
    zq = torch.randint(0, 16, sshape, generator=g)
    zpacked = O.pack_nibbles(zq)
    zfloat = (torch.randn(sshape, generator=g) * 5).to(od)
    fn = torch.ops.hpu.convert_from_int4 if signed else torch.ops.hpu.convert_from_uint4
    ofn = O.convert_from_int4 if signed else O.convert_from_uint4
    for zp in (None, zpacked, zfloat):
        r = fn(packed.cuda(), scale.cuda(), None if zp is None else zp.cuda(), od)
        assert _eq(r, ofn(packed, scale, zp, od)), (shape, group, None if zp is None else zp.dtype)


def test_kpacked_layout_matches_repacked_operator_layout(ops):
    """AutoGPTQ packs along K; the reference repacks on the host to the operator's layout
    (test_hpu_convert_from_int4.py:380-395).  The K-packed kernel must give the same matrix."""
    g = torch.Generator().manual_seed(3)
    K, N, group = 512, 256, 128
    w = torch.randint(0, 16, (K, N), generator=g)
    zq = torch.randint(0, 16, (K // group, N), generator=g)
    scale = (torch.rand(K // group, N, generator=g) * 0.015 + 0.005).to(torch.bfloat16)
    q_op = O.pack_nibbles(w)                                   # [K, N/8]
    q_k = O.pack_nibbles(w.t().contiguous()).t().contiguous()  # [K/8, N]
    z_op = O.pack_nibbles(zq)
    ref = O.convert_from_uint4(q_op, scale, z_op, torch.bfloat16)
    assert _eq(O.dequant_kpacked(q_k, scale, z_op), ref)
    a = torch.ops.hpu.convert_from_uint4(q_op.cuda(), scale.cuda(), z_op.cuda(), torch.bfloat16)
    b = torch.ops.b200q.dequant_kpacked(q_k.cuda(), scale.cuda(), z_op.cuda(), torch.bfloat16)
    assert _eq(a, ref) and _eq(b, ref)
    b0 = torch.ops.b200q.dequant_kpacked(q_k.cuda(), scale.cuda(), None, torch.float32)
    assert _eq(b0, O.dequant_kpacked(q_k, scale, None, torch.float32))


def test_full_size_weight_matrix(ops):
    """K = N = 8192, group 128 (the benchmark's shape): sampled rows bit-exact against the oracle,
    and a checksum identity: sum over the dequantised matrix of rows of one group equals
    scale * sum(q - zp) computed from integer sums."""
    g = torch.Generator(device="cuda").manual_seed(0)
    K = N = 8192
    packed = torch.randint(-2 ** 31, 2 ** 31 - 1, (K, N // 8), device="cuda", dtype=torch.int32, generator=g)
    scale = (torch.rand(K // 128, N, device="cuda", generator=g) * 0.015 + 0.005).to(torch.bfloat16)
    zp = torch.randint(-2 ** 31, 2 ** 31 - 1, (K // 128, N // 8), device="cuda", dtype=torch.int32, generator=g)
    out = torch.ops.hpu.convert_from_uint4(packed, scale, zp, torch.bfloat16)
    assert out.shape == (K, N) and out.dtype == torch.bfloat16
    rows = torch.tensor([0, 1, 127, 128, 129, 4095, 4096, 8191])
    for r in rows.tolist():
        grp = r // 128
        ref = O.convert_from_uint4(packed[r:r + 1].cpu(), scale[grp:grp + 1].cpu(), zp[grp:grp + 1].cpu(),
                                   torch.bfloat16)
        assert torch.equal(out[r:r + 1].cpu().float(), ref.float()), r
    # every value is (integer in [-15, 15]) * scale: dividing by the scale gives integers back
    ratio = out[:128].float() / scale[0].float()
    assert torch.all((ratio - ratio.round()).abs() < 0.26)  # bf16 rounding of the product: < 2^-8 * 15 * ...


# ---------------------------------------------------------------- fused W4A16 GEMM
def _w4_case(M, N, K, group, g, with_zp=True):
    w = torch.randint(0, 16, (K, N), generator=g)
    qw = O.pack_nibbles(w)
    scale = (torch.rand(K // group, N, generator=g) * 0.015 + 0.005).to(torch.bfloat16)
    zp = O.pack_nibbles(torch.randint(0, 16, (K // group, N), generator=g)) if with_zp else None
    x = torch.randn(M, K, generator=g).to(torch.bfloat16)
    return x, qw, scale, zp


@pytest.mark.parametrize("M", [1, 16, 17, 64, 128, 130, 384])
@pytest.mark.parametrize("N,K,group", [(256, 256, 128), (384, 512, 64), (1024, 2048, 128)])
def test_w4a16_matches_composition(ops, M, N, K, group):
    """out = x @ convert_from_uint4(...): the fused kernel against the oracle's composition, and
    (in fp32 output, where no output rounding hides anything) against the unfused GPU path."""
    g = torch.Generator().manual_seed(M * 31 + N)
    for with_zp in (True, False):
        x, qw, scale, zp = _w4_case(M, N, K, group, g, with_zp)
        zc = None if zp is None else zp.cuda()
        r = torch.ops.b200q.w4a16_gemm(x.cuda(), qw.cuda(), scale.cuda(), zc, group, False, torch.bfloat16)
        e = O.w4a16_gemm(x, qw, scale, zp, torch.bfloat16)
        assert r.dtype == torch.bfloat16 and r.shape == (M, N)
        assert O.rel_frobenius(r, e) <= 1e-2
        r32 = torch.ops.b200q.w4a16_gemm(x.cuda(), qw.cuda(), scale.cuda(), zc, group, False, torch.float32)
        wdq = torch.ops.hpu.convert_from_uint4(qw.cuda(), scale.cuda(), zc, torch.bfloat16)
        e32 = x.cuda().float() @ wdq.float()
        assert O.rel_frobenius(r32, e32) <= 2e-5
    assert ops.device_status() == 0


def test_w4a16_weight_layout_probe(ops):
    """One-hot activations read single rows of the dequantised weight matrix back through the
    tensor cores: any mistake in the 8x8 register transpose or the swizzled tile layout shows up
    as a wrong element, not as noise."""
    g = torch.Generator().manual_seed(5)
    N, K, group = 512, 512, 128
    _, qw, scale, zp = _w4_case(1, N, K, group, g)
    wdq = O.convert_from_uint4(qw, scale, zp, torch.bfloat16).float()
    for M in (16, 256):
        rows = (torch.arange(M) * 37) % K
        x = torch.zeros(M, K)
        x[torch.arange(M), rows] = 1.0
        r = torch.ops.b200q.w4a16_gemm(x.to(torch.bfloat16).cuda(), qw.cuda(), scale.cuda(), zp.cuda(), group, False,
                                       torch.float32)
        assert torch.equal(r.cpu(), wdq[rows]), M
    assert ops.device_status() == 0


def test_w4a16_full_size(ops):
    """K = N = 8192, group 128 (the benchmark's weight): M = 16 and M = 2048 against the unfused
    GPU composition on sampled rows, and two runs agree bit for bit (the split-K sum is ordered)."""
    g = torch.Generator(device="cuda").manual_seed(0)
    K = N = 8192
    qw = torch.randint(-2 ** 31, 2 ** 31 - 1, (K, N // 8), device="cuda", dtype=torch.int32, generator=g)
    scale = (torch.rand(K // 128, N, device="cuda", generator=g) * 0.015 + 0.005).to(torch.bfloat16)
    zp = torch.randint(-2 ** 31, 2 ** 31 - 1, (K // 128, N // 8), device="cuda", dtype=torch.int32, generator=g)
    wdq = torch.ops.hpu.convert_from_uint4(qw, scale, zp, torch.bfloat16)
    for M in (16, 2048):
        x = torch.randn(M, K, device="cuda", generator=g).to(torch.bfloat16)
        r1 = torch.ops.b200q.w4a16_gemm(x, qw, scale, zp, 128, False, torch.bfloat16)
        r2 = torch.ops.b200q.w4a16_gemm(x, qw, scale, zp, 128, False, torch.bfloat16)
        assert torch.equal(r1, r2)
        rows = torch.tensor([0, 1, M // 2, M - 1], device="cuda")
        e = (x[rows].double() @ wdq.double()).float()
        assert O.rel_frobenius(r1[rows], e) <= 1e-2
    assert ops.device_status() == 0


def test_gptq_repack_matches_reference_host_repack(ops):
    """AutoGPTQ qweight / qzeros -> operator layout on the device, bit for bit what the reference's
    own host-side helper produced (golden), and the repacked tensors dequantise to the GPTQ result."""
    z = np.load(os.path.join(GOLDEN, "int4.npz"))
    for i in range(int(z["n_gptq"])):
        k = f"a{i}"
        od = _DT[z[k + "_meta"][0]]
        is_zp = z[k + "_meta"][1] == "True"
        gq = torch.from_numpy(z[k + "_gptq_qweight"]).cuda()
        gz = torch.from_numpy(z[k + "_gptq_qzeros"]).cuda()
        qw, qz = torch.ops.b200q.gptq_repack(gq, gz)
        assert torch.equal(qw.cpu(), torch.from_numpy(z[k + "_qweight"])), k
        assert torch.equal(qz.cpu(), torch.from_numpy(z[k + "_qzeros"])), k
        sc = torch.from_numpy(z[k + "_scale"]).to(od).cuda()
        r = torch.ops.hpu.convert_from_uint4(qw, sc, qz if is_zp else None, od)
        assert torch.equal(r.cpu().float(), torch.from_numpy(z[k + "_ref"])), k
    # a larger matrix against the oracle's packers
    g = torch.Generator().manual_seed(8)
    K, N = 1024, 768
    w = torch.randint(0, 16, (K, N), generator=g)
    kpacked = O.pack_nibbles(w.t().contiguous()).t().contiguous()
    zq = torch.randint(0, 16, (K // 128, N), generator=g)
    qw, qz = torch.ops.b200q.gptq_repack(kpacked.cuda(), O.pack_nibbles((zq - 1) & 0xF).cuda())
    assert torch.equal(qw.cpu(), O.pack_nibbles(w)) and torch.equal(qz.cpu(), O.pack_nibbles(zq))


def test_w4a16_degenerate_k():
    """K = 32 (below the kernel's 64-deep k-block) is refused with an error, K = 0 gives zeros."""
    dev = "cuda"
    x = torch.randn(4, 32, device=dev).to(torch.bfloat16)
    qw = torch.zeros(32, 8, dtype=torch.int32, device=dev)
    sc = torch.ones(1, 64, dtype=torch.bfloat16, device=dev)
    with pytest.raises(RuntimeError):
        torch.ops.b200q.w4a16_gemm(x, qw, sc, None, 32, False, torch.bfloat16)
    from b200_hpu_ops import abi
    out = torch.full((4, 64), 7.0, dtype=torch.bfloat16, device=dev)
    rc = abi.lib.b200q_w4a16_gemm(abi.ptr(x), 0, abi.ptr(qw), abi.ptr(sc), None, abi.ZP_NONE, 0, 4, 64, 0, 64,
                                  abi.ptr(out), abi.BF16, 64, None, 0, abi.stream_ptr())
    assert rc == 0
    assert torch.count_nonzero(out).item() == 0


def _pack_k(w):
    """[K, N] nibble values -> AutoGPTQ layout [K/8, N]: nibble i of word (r, n) is w[8r + i, n]."""
    return O.pack_nibbles(w.t().contiguous()).t().contiguous()


@pytest.mark.parametrize("M", [1, 5, 8, 9, 16])
@pytest.mark.parametrize("N,K,group", [(512, 256, 128), (1024, 2048, 64), (512, 4096, 128), (1024, 8192, 128)])
@pytest.mark.parametrize("k_packed", [False, True])
def test_w4a16_few_tokens_kernel(ops, M, N, K, group, k_packed):
    """M <= 16 takes the streaming kernel (cluster-reduced, no scratch) for both weight layouts:
    fp32 output against the unfused GPU composition (same bf16 weights, fp32 sums), bf16 output
    against the oracle, and a one-hot probe that reads single weight rows back exactly."""
    if k_packed and K % 1024:
        pytest.skip("the AutoGPTQ-layout form of the kernel needs K % 1024 == 0")
    g = torch.Generator().manual_seed(M * 131 + N + K)
    for with_zp in (True, False):
        w = torch.randint(0, 16, (K, N), generator=g)
        qw = _pack_k(w) if k_packed else O.pack_nibbles(w)
        scale = (torch.rand(K // group, N, generator=g) * 0.015 + 0.005).to(torch.bfloat16)
        zp = O.pack_nibbles(torch.randint(0, 16, (K // group, N), generator=g)) if with_zp else None
        x = torch.randn(M, K, generator=g).to(torch.bfloat16)
        zc = None if zp is None else zp.cuda()
        assert ops.abi.lib.b200q_w4a16_workspace_bytes(M, N, K) == 0
        wdq = O.convert_from_uint4(O.pack_nibbles(w), scale, zp, torch.bfloat16)
        r32 = torch.ops.b200q.w4a16_gemm(x.cuda(), qw.cuda(), scale.cuda(), zc, group, k_packed, torch.float32)
        e32 = (x.double() @ wdq.double()).float()
        assert O.rel_frobenius(r32, e32) <= 2e-5
        r = torch.ops.b200q.w4a16_gemm(x.cuda(), qw.cuda(), scale.cuda(), zc, group, k_packed, torch.bfloat16)
        assert r.dtype == torch.bfloat16 and r.shape == (M, N)
        assert O.rel_frobenius(r, e32) <= 1e-2
        assert torch.equal(r, torch.ops.b200q.w4a16_gemm(x.cuda(), qw.cuda(), scale.cuda(), zc, group, k_packed, torch.bfloat16))
        rows = (torch.arange(M) * 397 + 11) % K
        hot = torch.zeros(M, K)
        hot[torch.arange(M), rows] = 1.0
        rh = torch.ops.b200q.w4a16_gemm(hot.to(torch.bfloat16).cuda(), qw.cuda(), scale.cuda(), zc, group, k_packed, torch.float32)
        assert torch.equal(rh.cpu(), wdq.float()[rows])
    assert ops.device_status() == 0


def test_w4a16_kpacked_many_tokens_goes_through_repack(ops):
    g = torch.Generator().manual_seed(77)
    M, N, K, group = 160, 512, 1024, 128
    w = torch.randint(0, 16, (K, N), generator=g)
    scale = (torch.rand(K // group, N, generator=g) * 0.015 + 0.005).to(torch.bfloat16)
    zp = O.pack_nibbles(torch.randint(0, 16, (K // group, N), generator=g))
    x = torch.randn(M, K, generator=g).to(torch.bfloat16)
    a = torch.ops.b200q.w4a16_gemm(x.cuda(), _pack_k(w).cuda(), scale.cuda(), zp.cuda(), group, True, torch.bfloat16)
    b = torch.ops.b200q.w4a16_gemm(x.cuda(), O.pack_nibbles(w).cuda(), scale.cuda(), zp.cuda(), group, False, torch.bfloat16)
    assert torch.equal(a, b)
