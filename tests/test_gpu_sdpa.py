"""hpu::fp8_sdpa_recomp_fwd on the GPU: the tcgen05 kernel (head dimension 128) and the plain kernel
(other head dimensions) against the CPU restatement (same quantisation points) and -- with the
bound the reference's own test uses for fp8 runs, atol 0.4
(tests/pytest_working/any_mode/FusedSDPA/test_hpu_sdpa_fp8.py:1028-1060) -- against plain attention
on the unquantised tensors, as that test does."""
import math

import pytest
import torch

from oracle import hpu_oracle as O

pytestmark = pytest.mark.gpu
E4M3 = torch.float8_e4m3fn


@pytest.fixture(autouse=True)
def _status():
    import b200_hpu_ops
    yield
    assert b200_hpu_ops.device_status() == 0


def _quant(x, amax_target=448.0):
    s = amax_target / x.abs().max()
    x8, _ = O.cast_to_fp8_v2(x.to(torch.bfloat16), s, False, False, E4M3)
    return x8, 1.0 / s


def _vanilla(q, k, v, mask, causal, scale):
    s = torch.matmul(q, k.transpose(-2, -1)) * scale
    if mask is not None:
        s = s.masked_fill(~mask, -1e30) if mask.dtype == torch.bool else s + mask.float()
    if causal:
        L, S = q.shape[-2], k.shape[-2]
        s = s.masked_fill(~torch.ones(L, S, dtype=torch.bool).tril(0), -1e30)
    p = torch.softmax(s, -1)
    return torch.matmul(p, v), p


def _run(q8, k8, v8, mask, causal, scale, dq, dk, dv, qs, qo, ds, bwd, amax, scalar):
    cu = lambda t: None if t is None else t.cuda()  # noqa: E731
    if scalar:
        f = lambda t: 0.0 if t is None else float(t)  # noqa: E731
        return torch.ops.hpu.fp8_sdpa_recomp_fwd.scalar(q8.cuda(), k8.cuda(), v8.cuda(), cu(mask), 0.0, scale, causal, bwd, "None",
                                                        f(dq), f(dk), f(dv), f(qs), f(qo), f(ds), amax, amax, None, "left")
    t = lambda x: None if x is None else torch.tensor([float(x)], dtype=torch.float32, device="cuda")  # noqa: E731
    return torch.ops.hpu.fp8_sdpa_recomp_fwd(q8.cuda(), k8.cuda(), v8.cuda(), cu(mask), 0.0, scale, causal, bwd, "None",
                                             t(dq), t(dk), t(dv), t(qs), t(qo), t(ds), amax, amax, None, "left")


CASES = [
    # B, Hq, Hkv, L, S, D, Dv, mask, causal
    (2, 4, 4, 256, 256, 128, 128, None, True),
    (1, 8, 2, 384, 384, 128, 128, None, True),         # grouped-query (5-D, as the reference's caller reshapes it)
    (2, 4, 1, 200, 333, 128, 128, "float_row", False),  # multi-query, ragged lengths, Bx1x1xS float mask
    (1, 2, 2, 128, 640, 128, 128, "bool_full", False),
    (2, 3, 3, 77, 150, 64, 64, None, True),             # plain kernel
    (1, 2, 2, 50, 260, 96, 80, "float_row", False),     # plain kernel, head_dim_v != head_dim_qk
    (3, 0, 0, 130, 130, 128, 128, None, False),         # 3-D tensors (no head dimension)
]


@pytest.mark.parametrize("B,Hq,Hkv,L,S,D,Dv,mask_kind,causal", CASES)
@pytest.mark.parametrize("fp8_out", [False, True])
def test_fp8_sdpa_recomp_fwd(B, Hq, Hkv, L, S, D, Dv, mask_kind, causal, fp8_out):
    g = torch.Generator().manual_seed(L * 7 + S + D)
    if Hq == 0:
        qs_, ks_, vs_ = (B, L, D), (B, S, D), (B, S, Dv)
    else:
        qs_, ks_, vs_ = (B, Hq, L, D), (B, Hkv, S, D), (B, Hkv, S, Dv)
    q, k, v = torch.randn(qs_, generator=g), torch.randn(ks_, generator=g), torch.randn(vs_, generator=g)
    q8, dq = _quant(q)
    k8, dk = _quant(k)
    v8, dv = _quant(v)
    scale = 1.0 / math.sqrt(D)
    mask = None
    if mask_kind == "float_row":
        keep = torch.randint(0, 2, (S,), generator=g).bool()
        keep[0] = True
        m1 = torch.zeros(S).masked_fill(~keep, -10000.0).to(torch.bfloat16)
        mask = m1.expand((B, 1, 1, S) if Hq else (B, 1, S))
    elif mask_kind == "bool_full":
        mask = torch.rand((B, Hq, L, S), generator=g) > 0.3
        mask[..., 0] = True
    q_scale_s, q_scale_o = 256.0, (16.0 if fp8_out else None)
    # grouped-query: the reference's Python caller reshapes to 5-D before the operator
    q8o, k8o, v8o, masko = q8, k8, v8, mask
    gqa = Hq and Hkv not in (1, Hq)
    if gqa:
        q8o = q8.reshape(B, Hkv, Hq // Hkv, L, D)
        k8o, v8o = k8.reshape(B, Hkv, 1, S, D), v8.reshape(B, Hkv, 1, S, Dv)
    for scalar in (False, True):
        out, m, linv, seed, amax_s, amax_o = _run(q8o, k8o, v8o, masko, causal, scale, dq, dk, dv, q_scale_s, q_scale_o, None,
                                                  True, True, scalar)
        e_out, e_m, e_linv, _, e_as, e_ao = O.fp8_sdpa_recomp_fwd(q8o, k8o, v8o, masko, 0.0, scale, causal, True, "None", dq, dk,
                                                                  dv, q_scale_s, q_scale_o, None, True, True)
        assert out.shape == e_out.shape and out.dtype == e_out.dtype
        assert m.shape == e_m.shape == linv.shape and m.dtype == torch.bfloat16
        of, ef = out.cpu().float(), e_out.float()
        if fp8_out:
            of, ef = of / q_scale_o, ef / q_scale_o
            assert O.rel_frobenius(of, ef) <= 4e-2      # one e4m3 step where a value sits on a tie
        else:
            assert O.rel_frobenius(of, ef) <= 5e-3, O.rel_frobenius(of, ef)
        assert torch.allclose(m.cpu().float(), e_m.float(), atol=2e-2, rtol=1e-2)
        assert torch.allclose(linv.cpu().float(), e_linv.float(), atol=1e-3, rtol=2e-2)
        assert abs(amax_s.item() - e_as.item()) <= 1e-3 * max(1.0, e_as.item())
        assert abs(amax_o.item() - e_ao.item()) <= 2e-2 * max(1.0, e_ao.item())
        # the reference test's own bound, against attention on the unquantised tensors
        kk, vv = k, v
        if Hq and Hkv != Hq:
            kk, vv = k.repeat_interleave(Hq // Hkv, 1), v.repeat_interleave(Hq // Hkv, 1)
        ref, _ = _vanilla(q, kk, vv, mask, causal, scale)
        got = of.reshape(ref.shape)
        assert torch.allclose(got, ref, rtol=1e-3, atol=0.4)


def test_fp8_sdpa_inference_outputs_and_checks():
    g = torch.Generator().manual_seed(1)
    q8, dq = _quant(torch.randn(1, 2, 128, 128, generator=g))
    k8, dk = _quant(torch.randn(1, 2, 128, 128, generator=g))
    out, m, linv, seed, amax_s, amax_o = _run(q8, k8, k8, None, True, 0.1, dq, dk, dk, None, None, None, False, False, False)
    assert out.dtype == torch.bfloat16 and m.shape == (1,) and linv.shape == (1,) and seed.shape == (1,)
    assert amax_s.item() == 0.0 and amax_o.item() == 0.0
    with pytest.raises(RuntimeError, match="dropout"):
        torch.ops.hpu.fp8_sdpa_recomp_fwd(q8.cuda(), k8.cuda(), k8.cuda(), None, 0.1, 0.1, True, False, "None", None, None, None,
                                          None, None, None, False, False, None, "left")
    with pytest.raises(RuntimeError, match="float8_e4m3fn"):
        torch.ops.hpu.fp8_sdpa_recomp_fwd(q8.cuda().to(torch.bfloat16), k8.cuda(), k8.cuda(), None, 0.0, 0.1, True, False, "None",
                                          None, None, None, None, None, None, False, False, None, "left")


def test_fp8_sdpa_long_sequence_both_kernels_agree(monkeypatch):
    """4096 keys: the tcgen05 kernel against the plain kernel through the C ABI (force_plain)."""
    import ctypes as C
    from b200_hpu_ops import abi
    g = torch.Generator(device="cuda").manual_seed(3)
    BH, L, S, D = 4, 512, 4096, 128
    q8 = torch.randn(BH, L, D, device="cuda", generator=g).mul(40).to(E4M3)
    k8 = torch.randn(BH, S, D, device="cuda", generator=g).mul(40).to(E4M3)
    v8 = torch.randn(BH, S, D, device="cuda", generator=g).mul(40).to(E4M3)
    outs = []
    for plain in (0, 1):
        out = torch.empty(BH, L, D, device="cuda", dtype=torch.bfloat16)
        a = abi.SdpaArgs()
        a.q, a.k, a.v, a.out, a.out_dtype = q8.data_ptr(), k8.data_ptr(), v8.data_ptr(), out.data_ptr(), abi.BF16
        a.BH, a.L, a.S, a.dqk, a.dv, a.kv_rep, a.causal = BH, L, S, D, D, 1, 1
        a.softmax_scale = 1.0 / math.sqrt(D)
        a.d_scale_q_host = a.d_scale_k_host = 1.0 / 40
        a.d_scale_v_host, a.q_scale_s_host, a.q_scale_o_host, a.d_scale_s_host = 1.0 / 40, 256.0, 1.0, 1.0
        a.force_plain = plain
        a.stream = torch.cuda.current_stream().cuda_stream
        abi.check(abi.lib.b200q_fp8_sdpa_fwd(C.byref(a)), "b200q_fp8_sdpa_fwd")
        outs.append(out)
    torch.cuda.synchronize()
    assert O.rel_frobenius(outs[0], outs[1]) <= 5e-3
