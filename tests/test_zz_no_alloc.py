"""b200q_w4a16_gemm_noalloc: the W4A16 GEMM for callers that may not allocate device memory
(a serving loop with a frozen memory plan, a plug-in inside another framework's callback, a host
binding without an allocator).  Its split-K scratch is a static array inside the library, so the
caller passes inputs and output only.

Checked through the C ABI against b200q_w4a16_gemm with a caller-provided workspace: the two
entry points run the same kernels in the same order, so the results must be identical; the
check is repeated on a second call because the static scratch keeps the first call's contents.
This file sorts last on purpose: a run that stops at the first failure has then already run
every other test."""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def _case(M, N, K, group, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    qw = torch.randint(-2 ** 31, 2 ** 31 - 1, (K, N // 8), device="cuda", dtype=torch.int32, generator=g)
    scale = (torch.rand(K // group, N, device="cuda", generator=g) * 0.015 + 0.005).to(torch.bfloat16)
    zp = torch.randint(-2 ** 31, 2 ** 31 - 1, (K // group, N // 8), device="cuda", dtype=torch.int32, generator=g)
    x = torch.randn(M, K, device="cuda", generator=g).to(torch.bfloat16)
    return x, qw, scale, zp


def _with_workspace(abi, x, qw, scale, zp, group, out):
    M, K = x.shape
    N = qw.shape[1] * 8
    need = abi.lib.b200q_w4a16_workspace_bytes(M, N, K)
    ws = torch.empty(max(need, 16), dtype=torch.uint8, device="cuda")
    abi.check(abi.lib.b200q_w4a16_gemm(abi.ptr(x), K, abi.ptr(qw), abi.ptr(scale), abi.ptr(zp), abi.ZP_PACKED, 0, M, N, K,
                                       group, abi.ptr(out), abi.DTYPE[out.dtype], N, abi.ptr(ws), need, abi.stream_ptr()),
              "b200q_w4a16_gemm")
    return need


def _no_alloc(abi, x, qw, scale, zp, group, out):
    M, K = x.shape
    N = qw.shape[1] * 8
    return abi.lib.b200q_w4a16_gemm_noalloc(abi.ptr(x), K, abi.ptr(qw), abi.ptr(scale), abi.ptr(zp), abi.ZP_PACKED, 0, M, N,
                                            K, group, abi.ptr(out), abi.DTYPE[out.dtype], N, abi.stream_ptr())


def test_noalloc_matches_workspace_entry_twice_in_a_row():
    import b200_hpu_ops
    from b200_hpu_ops import abi
    from oracle import hpu_oracle as O

    # two different problems back to back, both on the split-K path (so the scratch is really used;
    # 16 tokens or fewer would take the kernel that reduces inside its clusters and needs none)
    for call, (M, N, K, group, dt) in enumerate([(24, 2048, 4096, 128, torch.bfloat16), (21, 1024, 2048, 64, torch.float32)]):
        x, qw, scale, zp = _case(M, N, K, group, seed=100 + call)
        ref = torch.empty(M, N, dtype=dt, device="cuda")
        need = _with_workspace(abi, x, qw, scale, zp, group, ref)
        assert need > 0, "this shape must exercise the scratch"
        got = torch.full((M, N), float("nan"), dtype=dt, device="cuda")
        assert _no_alloc(abi, x, qw, scale, zp, group, got) == 0
        torch.cuda.synchronize()
        assert torch.equal(got, ref), f"call {call}: static-scratch result differs from the workspace result"
        # and both agree with the unfused composition within the GEMM tolerance of the other tests
        wdq = torch.ops.hpu.convert_from_uint4(qw, scale, zp, torch.bfloat16)
        assert O.rel_frobenius(got, (x.double() @ wdq.double()).float()) <= 1e-2
    # a shape that needs no scratch goes through as well
    x, qw, scale, zp = _case(256, 512, 512, 128, seed=7)
    ref = torch.empty(256, 512, dtype=torch.bfloat16, device="cuda")
    assert _with_workspace(abi, x, qw, scale, zp, 128, ref) == 0
    got = torch.empty_like(ref)
    assert _no_alloc(abi, x, qw, scale, zp, 128, got) == 0
    torch.cuda.synchronize()
    assert torch.equal(got, ref)
    assert b200_hpu_ops.device_status() == 0


def test_noalloc_rejects_what_does_not_fit():
    from b200_hpu_ops import abi
    M, N, K = 128, 8192, 8192   # would need 32 MiB of scratch
    assert abi.lib.b200q_w4a16_workspace_bytes(M, N, K) > (8 << 20)
    x, qw, scale, zp = _case(M, N, K, 128, seed=1)
    out = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    rc = _no_alloc(abi, x, qw, scale, zp, 128, out)
    assert rc == -4 and b"maximum" in abi.lib.b200q_strerror(rc)
    assert abi.lib.b200q_w4a16_gemm_noalloc(None, 0, None, None, None, 0, 0, 4, 8, 64, 64, None, abi.BF16, 8, None) == -1
