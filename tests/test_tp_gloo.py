"""The tensor-parallel MLP's partitioning and collective on CPU ranks (gloo, world size 2 and 4):
every rank runs the real TpFp8Mlp control flow with a stand-in for the operators (the CPU
oracle), and the all-reduced result must match the single-device oracle MLP."""
import os
import socket
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import ROOT


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _make_problem(T=48, d=64, f=128, seed=0):
    from oracle import hpu_oracle as O
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


class _OracleOps:
    """Stand-in for torch.ops.hpu on CPU ranks (test only)."""

    @staticmethod
    def cast_to_fp8_v2(x, scale, sr, is_amax, dtype, scale_shape=None):
        from oracle import hpu_oracle as O
        return O.cast_to_fp8_v2(x, scale, sr, is_amax, dtype, scale_shape)

    @staticmethod
    def fp8_gemm_v2(A, tA, B, tB, D, od, sa, sb, bias, acc, shape=None):
        from oracle import hpu_oracle as O
        return O.fp8_gemm_v2(A, tA, B, tB, D, od, sa, sb, bias, acc, shape)


def _worker(rank, world, port, q):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "gaudi-pytorch-bridge_b200"))
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        # tp_mlp is imported as a plain module: the package __init__ would load the CUDA libraries
        import importlib.util
        spec = importlib.util.spec_from_file_location(
            "tp_mlp", os.path.join(ROOT, "gaudi-pytorch-bridge_b200", "b200_hpu_ops", "tp_mlp.py"))
        tp_mlp = importlib.util.module_from_spec(spec)
        sys.modules["tp_mlp"] = tp_mlp
        spec.loader.exec_module(tp_mlp)
        from oracle import hpu_oracle as O
        x, wg8, wu8, wd8, sg, su, sd, xs, acs = _make_problem()
        shard = tp_mlp.shard_mlp(wg8, wu8, wd8, sg, su, sd, world, rank)
        assert shard.w_gate_up.shape == (2 * 128 // world, 64) and shard.w_down.shape == (64, 128 // world)
        mlp = tp_mlp.TpFp8Mlp(shard, xs, acs, row_blocks=3, ops=_OracleOps)
        y = mlp(x.clone())
        ref = O.fp8_swiglu_mlp(x, wg8, wu8, wd8, sg, su, sd, xs, acs)
        err = O.rel_frobenius(y, ref)
        # every rank holds the same reduced result
        gathered = [torch.empty_like(y) for _ in range(world)]
        dist.all_gather(gathered, y)
        same = all(torch.equal(gathered[0], t) for t in gathered)
        q.put((rank, err, same, tuple(y.shape)))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_tp_mlp_on_gloo_ranks(world):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = [q.get(timeout=180) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, err, same, shape in res:
        assert shape == (48, 64)
        assert same, "ranks disagree after the all-reduce"
        assert err <= 1e-2, (rank, err)   # bf16 partial sums round differently from the single-device sum


def test_shard_bounds_and_errors():
    import importlib.util
    spec = importlib.util.spec_from_file_location(
        "tp_mlp_x", os.path.join(ROOT, "gaudi-pytorch-bridge_b200", "b200_hpu_ops", "tp_mlp.py"))
    m = importlib.util.module_from_spec(spec)
    sys.modules["tp_mlp_x"] = m
    spec.loader.exec_module(m)
    assert m.shard_bounds(28672, 8, 3) == (3 * 3584, 4 * 3584)
    assert m.shard_bounds(14336, 1, 0) == (0, 14336)
    with pytest.raises(ValueError):
        m.shard_bounds(10, 4, 0)
    assert m.mlp_flops(8192, 8192, 28672) == pytest.approx(11.545e12, rel=1e-3)


# ---------------------------------------------------------------------------- sharded current-scaling cast
class _OracleB200Q:
    """Stand-in for torch.ops.b200q on CPU ranks (test only)."""

    @staticmethod
    def amax(x):
        return x.detach().abs().max().float().reshape(())

    @staticmethod
    def scale_from_amax_(scale, amax, fp8_max, pow2=True, margin=0):
        from oracle import hpu_oracle as O
        scale.copy_(O.scale_from_amax(amax, scale, fp8_max, pow2, margin).reshape(scale.shape))
        return scale


def _scaling_worker(rank, world, port, q):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import importlib.util
        spec = importlib.util.spec_from_file_location(
            "scaling", os.path.join(ROOT, "gaudi-pytorch-bridge_b200", "b200_hpu_ops", "scaling.py"))
        scaling = importlib.util.module_from_spec(spec)
        sys.modules["scaling"] = scaling
        spec.loader.exec_module(scaling)
        from oracle import hpu_oracle as O
        g = torch.Generator().manual_seed(3)
        x = (torch.randn(64, 96, generator=g) * 3).to(torch.bfloat16)
        x[37, 5] = 41.0  # the global amax sits in one rank's rows only
        rows = 64 // world
        mine = x[rank * rows:(rank + 1) * rows].contiguous()
        out, scale, amax = scaling.current_scaling_cast(mine, torch.float8_e4m3fn, group=dist.group.WORLD,
                                                        ops=(_OracleB200Q, _OracleOps))
        # the unsharded cast on one device
        full_scale = O.scale_from_amax(x.abs().max().float(), torch.ones(()), 448.0, True)
        full, _ = O.cast_to_fp8_v2(x, full_scale.reshape(1), False, False, torch.float8_e4m3fn, [1])
        same = torch.equal(out.view(torch.uint8), full[rank * rows:(rank + 1) * rows].view(torch.uint8))
        q.put((rank, float(amax), float(scale), float(full_scale), same))
    finally:
        dist.destroy_process_group()


def test_sharded_current_scaling_uses_the_global_amax():
    """Rows split over 2 gloo ranks: one 4-byte MAX all-reduce makes the amax global, both ranks
    derive the same scale, and the shards are the bytes of the unsharded cast."""
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_scaling_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    try:
        res = [q.get(timeout=180) for _ in range(world)]
        for p in procs:
            p.join(timeout=60)
    finally:
        for p in procs:
            if p.is_alive():
                p.terminate()
    for rank, amax, scale, full_scale, same in res:
        assert amax == 41.0 and scale == full_scale == 8.0, (rank, amax, scale, full_scale)
        assert same, rank
