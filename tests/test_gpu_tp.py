"""The FP8 SwiGLU MLP on the GPU: single device against the oracle, and (when the box has two or
more GPUs) tensor-parallel over NCCL ranks against the same oracle."""
import os
import socket
import sys

import pytest
import torch

from conftest import ROOT
from oracle import hpu_oracle as O

pytestmark = pytest.mark.gpu


def _problem(T, d, f, seed=0):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(T, d, generator=g).to(torch.bfloat16)

    def q(w):
        s = 448.0 / w.abs().amax(dim=1, keepdim=True)
        w8, _ = O.cast_to_fp8_v2(w.to(torch.bfloat16), s, False, False, torch.float8_e4m3fn, list(s.shape))
        return w8, (1.0 / s).reshape(-1).float()

    wg8, sg = q(torch.randn(f, d, generator=g) * 0.05)
    wu8, su = q(torch.randn(f, d, generator=g) * 0.05)
    wd8, sd = q(torch.randn(d, f, generator=g) * 0.05)
    return x, wg8, wu8, wd8, sg, su, sd, 448.0 / 5.0, 448.0 / 2.0


def test_mlp_single_device_matches_oracle():
    import b200_hpu_ops
    from b200_hpu_ops import tp_mlp
    x, wg8, wu8, wd8, sg, su, sd, xs, acs = _problem(256, 512, 1024)
    shard = tp_mlp.shard_mlp(wg8.cuda(), wu8.cuda(), wd8.cuda(), sg.cuda(), su.cuda(), sd.cuda(), 1, 0)
    ref = O.fp8_swiglu_mlp(x, wg8, wu8, wd8, sg, su, sd, xs, acs)
    for fused in (True, False):
        y = tp_mlp.TpFp8Mlp(shard, xs, acs, fused_swiglu=fused)(x.cuda())
        assert y.shape == ref.shape and y.dtype == torch.bfloat16
        assert O.rel_frobenius(y, ref) <= 1e-2
    assert b200_hpu_ops.device_status() == 0


@pytest.mark.parametrize("T", [64, 256, 300])
def test_fused_gate_up_swiglu_is_bit_identical(T):
    """The gate/up GEMM with SwiGLU + cast in its epilogue (interleaved weights) against the two
    operators: same e4m3 bytes, hence the same MLP output bit for bit.  T = 64 has no fused kernel
    and takes the operator's own composition."""
    import b200_hpu_ops
    from b200_hpu_ops import tp_mlp
    x, wg8, wu8, wd8, sg, su, sd, xs, acs = _problem(T, 512, 1024, seed=T)
    args = (wg8.cuda(), wu8.cuda(), wd8.cuda(), sg.cuda(), su.cuda(), sd.cuda(), 1, 0)
    plain = tp_mlp.TpFp8Mlp(tp_mlp.shard_mlp(*args), xs, acs)
    shard_i = tp_mlp.shard_mlp(*args, interleave=True)
    fused = tp_mlp.TpFp8Mlp(shard_i, xs, acs, fused_gate_up=True)
    h_plain = plain.activation(plain.gate_up(x.cuda()))
    x8, _ = torch.ops.hpu.cast_to_fp8_v2(x.cuda(), xs, False, False, torch.float8_e4m3fn)
    h_fused = torch.ops.b200q.fp8_gemm_swiglu_cast(x8, shard_i.w_gate_up, fused._xs_inv, shard_i.s_gate_up_inv, acs)
    assert h_fused.shape == h_plain.shape == (T, 1024)
    assert torch.equal(h_fused.view(torch.uint8), h_plain.view(torch.uint8))
    assert torch.equal(fused(x.cuda()), plain(x.cuda()))
    assert b200_hpu_ops.device_status() == 0


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, q):
    """One NCCL rank: the interleaved gate/up shard with the SwiGLU + cast in the GEMM epilogue --
    the configuration bench.py's mlp record times -- against the oracle, plus the bytes of the
    e4m3 intermediate against the same columns computed without sharding."""
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "gaudi-pytorch-bridge_b200"))
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    import torch.distributed as dist
    inited = False
    try:
        torch.cuda.set_device(rank)
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
        inited = True
        import b200_hpu_ops
        from b200_hpu_ops import tp_mlp
        T, d, f = 1024, 512, 2048  # 1024 tokens: whole 128-row tiles per rank up to 8 ranks
        x, wg8, wu8, wd8, sg, su, sd, xs, acs = _problem(T, d, f)
        dev = torch.device("cuda", rank)
        args = (wg8.to(dev), wu8.to(dev), wd8.to(dev), sg.to(dev), su.to(dev), sd.to(dev))
        ref = O.fp8_swiglu_mlp(x, wg8, wu8, wd8, sg, su, sd, xs, acs)
        errs = []
        for comm in COMM_MODES:
            shard = tp_mlp.shard_mlp(*args, world, rank, interleave=True)
            mlp = tp_mlp.TpFp8Mlp(shard, xs, acs, row_blocks=4, fused_gate_up=True, comm=comm)
            full = tp_mlp.TpFp8Mlp(tp_mlp.shard_mlp(*args, 1, 0, interleave=True), xs, acs, fused_gate_up=True)
            lo, hi = tp_mlp.shard_bounds(f, world, rank)
            h_mine, h_full = mlp.hidden(x.to(dev)), full.hidden(x.to(dev))
            same = torch.equal(h_mine.view(torch.uint8), h_full[:, lo:hi].view(torch.uint8))
            for _ in range(2):  # twice: buffers and flags of the first call are reused by the second
                y = mlp(x.to(dev)).clone()
            torch.cuda.synchronize()
            errs.append((comm, float(O.rel_frobenius(y, ref)), same))
        # sharded current-scaling cast: rows split over the ranks, one MAX all-reduce of the amax,
        # and the shards must be the bytes of the unsharded cast
        from b200_hpu_ops import scaling
        xr = (x.float() * 3).to(torch.bfloat16).to(dev)
        rows = T // world
        o_sh, sc_sh, _ = scaling.current_scaling_cast(xr[rank * rows:(rank + 1) * rows].contiguous(), group=dist.group.WORLD)
        o_full, sc_full, _ = scaling.current_scaling_cast(xr)
        torch.cuda.synchronize()
        cast_ok = bool(torch.equal(o_sh.view(torch.uint8), o_full[rank * rows:(rank + 1) * rows].view(torch.uint8))
                       and torch.equal(sc_sh, sc_full))
        errs.append(("sharded_cast", 0.0 if cast_ok else 1.0, cast_ok))
        q.put((rank, errs, b200_hpu_ops.device_status()))
    except Exception as e:  # report instead of leaving the parent waiting on the queue
        q.put((rank, repr(e), -1))
    finally:
        if inited:
            dist.destroy_process_group()


COMM_MODES = ("nccl", "fused")


@pytest.mark.parametrize("world", [2, 4, 8])
def test_mlp_tensor_parallel_nccl(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    try:
        res = [q.get(timeout=300) for _ in range(world)]
        for p in procs:
            p.join(timeout=120)
    finally:
        for p in procs:  # never leave a rank behind inside a collective, holding its GPU
            if p.is_alive():
                p.terminate()
                p.join(timeout=10)
                if p.is_alive():
                    p.kill()
    for rank, errs, status in res:
        assert status == 0, (rank, errs)
        for comm, err, same in errs:
            assert same, (rank, comm, "e4m3 intermediate differs from the unsharded computation")
            assert err <= 1e-2, (rank, comm, err)
    for p in procs:
        assert p.exitcode == 0


@pytest.mark.parametrize("tp", [2, 4, 8])
@pytest.mark.parametrize("N", [512, 704])
def test_routed_gemm_and_reduce_bcast_on_one_device(tp, N):
    """The two kernels of the fused collective with the ranks emulated on one GPU: `tp` row-parallel
    GEMMs (one K-shard each) route their partial sums into per-owner staging buffers, then every
    owner adds the slots and writes its rows into all outputs.  Checked against the sum of the
    bf16 partial products formed with the ordinary (unrouted) GEMM, and against the oracle."""
    import b200_hpu_ops
    from b200_hpu_ops import abi
    T, Kf = 1024, 256 * tp
    rows = T // tp
    g = torch.Generator(device="cuda").manual_seed(tp * 7 + N)
    h8 = torch.randn(T, Kf, device="cuda", generator=g).clamp(-3, 3).mul(50).to(torch.float8_e4m3fn)
    w8 = torch.randn(N, Kf, device="cuda", generator=g).clamp(-3, 3).mul(50).to(torch.float8_e4m3fn)
    sb = torch.rand(N, device="cuda", generator=g) * 1e-4 + 1e-4
    stages = [torch.full((tp, rows, N), float("nan"), device="cuda", dtype=torch.bfloat16) for _ in range(tp)]
    outs = [torch.full((T, N), float("nan"), device="cuda", dtype=torch.bfloat16) for _ in range(tp)]
    partials = []
    for r in range(tp):
        hs, ws = h8[:, r * 256:(r + 1) * 256].contiguous(), w8[:, r * 256:(r + 1) * 256].contiguous()
        abi.fp8_gemm_nt(hs, ws, torch.bfloat16, 0.01, sb, None, route=([s.data_ptr() for s in stages], rows, r * rows))
        partials.append(abi.fp8_gemm_nt(hs, ws, torch.bfloat16, 0.01, sb, None))
    # slot r of owner i holds rank r's partial sums of the rows owner i owns, bit for bit
    for i in range(tp):
        for r in range(tp):
            assert torch.equal(stages[i][r], partials[r][i * rows:(i + 1) * rows]), (i, r)
    for i in range(tp):
        abi.tp_reduce_bcast(stages[i], [o.data_ptr() for o in outs], i, rows, N)
    torch.cuda.synchronize()
    acc = partials[0].float()
    for pr in partials[1:]:
        acc = acc + pr.float()   # fp32, in rank order
    want = acc.to(torch.bfloat16)  # one rounding
    for o in outs:
        assert torch.equal(o, want)
    ref = O.fp8_gemm_v2(h8.cpu(), False, w8.cpu(), True, None, torch.bfloat16, torch.tensor(0.01), sb.cpu(), None, False, [1, N])
    assert O.rel_frobenius(outs[0], ref) <= 1e-2
    assert b200_hpu_ops.device_status() == 0
