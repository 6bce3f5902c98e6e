"""Tensor-parallel FP8 SwiGLU MLP built from the hpu::* operators.

    y = down( fp8( silu(x8 @ Wg^T) * (x8 @ Wu^T) ) )          x8 = fp8(x * x_scale)

Sharding over `tp` ranks (one process per GPU):
* gate and up projections are column-parallel: rank r holds rows [r*f/tp, (r+1)*f/tp) of
  W_gate and W_up ([ffn, d_model], K-major) with their per-output-channel scale_inv slices; the
  activations are replicated; no collective.  The two shards are stacked into one [2f/tp, d]
  weight so that gate and up come out of a single fp8_gemm_v2 call.
* the down projection is row-parallel: rank r holds columns [r*f/tp, (r+1)*f/tp) of W_down
  ([d_model, ffn]) -- a [d, f/tp] K-major shard -- and produces a full-size [tokens, d] partial
  sum; one SUM all-reduce over the ranks finishes it.  The all-reduce is issued per block of
  token rows so that the reduction of block i overlaps the GEMM of block i+1 (the
  reference's collective is a chunked hcclAllReduce on a network stream,
  python_packages/habana_frameworks/torch/distributed/hccl/process_group_hccl_base.cpp:412-497).
* activation scales are per tensor and static (given), so no amax exchange sits on the path.

The operator namespace is a constructor argument so that the partitioning and the collective
can be exercised on CPU ranks (gloo) with a stand-in for the operators; the default is the
CUDA implementation registered by this package, and nothing here falls back to anything else.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional

import torch

E4M3 = torch.float8_e4m3fn


@dataclass
class MlpShard:
    """One rank's weights.  w_gate_up: e4m3 [2*f_local, d]; w_down: e4m3 [d, f_local]."""
    w_gate_up: torch.Tensor
    s_gate_up_inv: torch.Tensor  # fp32 [2*f_local]
    w_down: torch.Tensor
    s_down_inv: torch.Tensor     # fp32 [d]
    f_local: int


def shard_bounds(n: int, tp: int, rank: int):
    """Contiguous, equal shards; n must divide evenly (28672 / 8 = 3584 = 14 x 256 stays tile-aligned)."""
    if n % tp:
        raise ValueError(f"dimension {n} does not divide over {tp} ranks")
    step = n // tp
    return rank * step, (rank + 1) * step


def interleave_blocks(gate: torch.Tensor, up: torch.Tensor, block: int = 128) -> torch.Tensor:
    """[f, ...] gate and up -> [2f, ...] with blocks of `block` gate rows followed by the `block` up rows of
    the same hidden units: the layout whose 256-row tiles hold both halves of a SwiGLU."""
    f = gate.shape[0]
    if f % block:
        raise ValueError(f"hidden size {f} is not a multiple of {block}")
    g = gate.reshape(f // block, 1, block, *gate.shape[1:])
    u = up.reshape(f // block, 1, block, *up.shape[1:])
    return torch.cat([g, u], dim=1).reshape(2 * f, *gate.shape[1:]).contiguous()


def shard_mlp(w_gate8, w_up8, w_down8, s_gate_inv, s_up_inv, s_down_inv, tp: int, rank: int,
              interleave: bool = False) -> MlpShard:
    """Slice full e4m3 weights ([f, d], [f, d], [d, f]) and their scale_inv vectors for one rank.
    interleave=True stores gate and up rows in alternating blocks of 128 (see interleave_blocks) so that
    the gate/up GEMM can apply the SwiGLU in its epilogue (TpFp8Mlp(fused_gate_up=True))."""
    f = w_gate8.shape[0]
    lo, hi = shard_bounds(f, tp, rank)
    g8, u8 = w_gate8[lo:hi].view(torch.uint8), w_up8[lo:hi].view(torch.uint8)
    if interleave:
        gu = interleave_blocks(g8, u8).view(E4M3)
        sgu = interleave_blocks(s_gate_inv[lo:hi].float(), s_up_inv[lo:hi].float())
    else:
        gu = torch.cat([g8, u8], dim=0).view(E4M3).contiguous()
        sgu = torch.cat([s_gate_inv[lo:hi], s_up_inv[lo:hi]]).float().contiguous()
    wd = w_down8.view(torch.uint8)[:, lo:hi].contiguous().view(E4M3)
    return MlpShard(gu, sgu, wd, s_down_inv.float().contiguous(), hi - lo)


class PeerBuffers:
    """Two bf16 [tokens, d] buffers per rank that every rank of the group can address: `stage`
    (slot s of rank r = rank s's partial sums of the token rows r owns) and `out` (the finished
    result).  Allocated and exchanged through torch's symmetric-memory allocator (CUDA virtual
    memory handles passed between the processes, peer access over NVLink); the kernels see plain
    device pointers.  barrier() is a kernel on the current stream that returns once every rank of
    the group has reached it."""

    def __init__(self, tokens: int, d: int, device, group=None):
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm

        group = group if group is not None else dist.group.WORLD
        self.tp, self.rank = dist.get_world_size(group), dist.get_rank(group)
        if tokens % (self.tp * 128):
            raise ValueError(f"{tokens} tokens do not split into {self.tp} blocks of whole 128-row tiles")
        self.tokens, self.d, self.rows = tokens, d, tokens // self.tp
        self.stage = symm.empty(tokens, d, dtype=torch.bfloat16, device=device)
        self.out = symm.empty(tokens, d, dtype=torch.bfloat16, device=device)
        self._hs = symm.rendezvous(self.stage, group.group_name)
        self._ho = symm.rendezvous(self.out, group.group_name)
        self.stage_ptrs = [int(p) for p in self._hs.buffer_ptrs]
        self.out_ptrs = [int(p) for p in self._ho.buffer_ptrs]

    def barrier(self):
        # (the wait inside gives up after 20 s instead of spinning for ever on a rank that died)
        self._hs.barrier(0, 20000)


class TpFp8Mlp:
    """comm: how the row-parallel partial sums become the result at tp > 1.
    "nccl"   one NCCL bf16 SUM all-reduce per block of token rows, issued asynchronously so that
             block i's reduction overlaps block i+1's down-projection GEMM;
    "fused"  the down-projection GEMM writes each 128-row block of its partial sums straight into
             the staging buffer of the rank that owns those token rows (routed output: peer
             stores over NVLink from the GEMM's epilogue, tile by tile while the main loop
             runs), then every rank adds the tp partial sums of its rows in fp32 and writes the
             result into all ranks' outputs (b200q_tp_reduce_bcast).  One GEMM launch for all
             tokens, no NCCL call on the path; two barriers across the ranks per forward.  The
             result is returned in a buffer that the next forward overwrites;
    "auto"   "fused" on CUDA ranks when tokens divide into tp blocks of whole tiles, else "nccl"."""

    def __init__(self, shard: MlpShard, x_scale: float, act_scale: float, group=None, row_blocks: int = 8,
                 ops=None, fused_swiglu: bool = True, fused_gate_up: bool = False, comm: str = "auto"):
        self.s = shard
        self.x_scale = float(x_scale)
        self.act_scale = float(act_scale)
        self.group = group
        self.row_blocks = int(row_blocks)
        self.ops = ops if ops is not None else torch.ops.hpu
        self.fused_swiglu = fused_swiglu and ops is None
        # the shard's gate/up weights are interleaved (shard_mlp(..., interleave=True)): SwiGLU and the
        # cast run in the GEMM's epilogue and the bf16 [tokens, 2f] intermediate is never written
        self.fused_gate_up = fused_gate_up and ops is None
        if comm not in ("auto", "nccl", "fused"):
            raise ValueError(f"unknown comm mode {comm!r}")
        self.comm = comm
        self._peer: Optional[PeerBuffers] = None
        self._no_peer_buffers = False  # comm="auto": the ranks could not map each other's memory
        self.skip_collective = False  # measurement only: leaves the partial sums unreduced
        dev = shard.w_gate_up.device
        self._xs_inv = torch.tensor(1.0 / self.x_scale, dtype=torch.float32, device=dev)
        self._as_inv = torch.tensor(1.0 / self.act_scale, dtype=torch.float32, device=dev)

    def _mode(self, tp: int, tokens: int) -> str:
        if tp == 1:
            return "none"
        can_fuse = self.ops is torch.ops.hpu and tokens % (tp * 128) == 0 and tokens // tp >= 128 and tokens > 128
        if self.comm == "fused" and not can_fuse:
            raise ValueError(f"comm='fused' needs CUDA operators and tokens divisible into {tp} blocks of whole 128-row tiles")
        if self.comm == "auto" and self._no_peer_buffers:
            return "nccl"
        return "fused" if (self.comm in ("auto", "fused") and can_fuse) else "nccl"

    def describe(self, tp: int, tokens: int = 8192) -> str:
        mode = self._mode(tp, tokens)
        if mode == "none":
            return "tp1: one device, no collective"
        if mode == "fused":
            return (f"tp{tp}: column-parallel gate/up, row-parallel down whose epilogue stores each partial-sum block into "
                    f"its owner's memory over NVLink, then fp32 reduce + broadcast by the owners (no NCCL on the path)")
        return (f"tp{tp}: column-parallel gate/up, row-parallel down, NCCL bf16 all-reduce in {self.row_blocks} row "
                f"blocks overlapping the down-projection GEMMs")

    def launches_per_step(self, tp: int, tokens: int = 8192) -> int:
        """Kernels of this library per forward (NCCL's and the barrier's kernels are not counted)."""
        head = 2 if self.fused_gate_up else 3  # cast, gate/up GEMM (+ SwiGLU/cast kernel)
        mode = self._mode(tp, tokens)
        return head + (1 if mode == "none" else 2 if mode == "fused" else self.row_blocks)

    # -- the three local stages ------------------------------------------------------------
    def gate_up(self, x: torch.Tensor) -> torch.Tensor:
        x8, _ = self.ops.cast_to_fp8_v2(x, self.x_scale, False, False, E4M3)
        n = self.s.w_gate_up.shape[0]
        return self.ops.fp8_gemm_v2(x8, False, self.s.w_gate_up, True, None, torch.bfloat16, self._xs_inv,
                                    self.s.s_gate_up_inv, None, False, [1, n])

    def activation(self, gu: torch.Tensor) -> torch.Tensor:
        f = self.s.f_local
        if self.fused_swiglu:
            h8, _ = torch.ops.b200q.swiglu_cast_fp8(gu[:, :f], gu[:, f:], self.act_scale, False)
            return h8
        h = (torch.nn.functional.silu(gu[:, :f].float()) * gu[:, f:].float()).to(torch.bfloat16)
        h8, _ = self.ops.cast_to_fp8_v2(h, self.act_scale, False, False, E4M3)
        return h8

    def hidden(self, x: torch.Tensor) -> torch.Tensor:
        """e4m3 [tokens, f_local]: this rank's columns of cast(silu(gate) * up)."""
        if self.fused_gate_up:
            x8, _ = self.ops.cast_to_fp8_v2(x, self.x_scale, False, False, E4M3)
            return torch.ops.b200q.fp8_gemm_swiglu_cast(x8, self.s.w_gate_up, self._xs_inv, self.s.s_gate_up_inv, self.act_scale)
        return self.activation(self.gate_up(x))

    def down_partial(self, h8: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        d = self.s.w_down.shape[0]
        if out is not None and self.ops is torch.ops.hpu:
            # write straight into the caller's row block (the operator itself always allocates)
            from . import abi
            return abi.fp8_gemm_nt(h8, self.s.w_down, torch.bfloat16, 1.0 / self.act_scale, self.s.s_down_inv, None, out=out)
        r = self.ops.fp8_gemm_v2(h8, False, self.s.w_down, True, None, torch.bfloat16, self._as_inv, self.s.s_down_inv,
                                 None, False, [1, d])
        if out is not None:
            out.copy_(r)
            return out
        return r

    # -- forward -----------------------------------------------------------------------------
    def forward(self, x: torch.Tensor) -> torch.Tensor:
        import torch.distributed as dist

        h8 = self.hidden(x)
        tp = dist.get_world_size(self.group) if (dist.is_available() and dist.is_initialized()) else 1
        if tp == 1:
            return self.down_partial(h8)
        if self._mode(tp, h8.shape[0]) == "fused" and self._ensure_peer_buffers(h8):
            return self._down_fused(h8)
        rows = h8.shape[0]
        nblk = max(1, min(self.row_blocks, rows))
        step = (rows + nblk - 1) // nblk
        out = torch.empty(rows, self.s.w_down.shape[0], dtype=torch.bfloat16, device=h8.device)
        works: List = []
        for b in range(nblk):
            lo, hi = b * step, min(rows, (b + 1) * step)
            if lo >= hi:
                break
            self.down_partial(h8[lo:hi], out[lo:hi])
            # the collective of this block runs on the communicator's stream while the next
            # block's GEMM runs on the compute stream
            if not self.skip_collective:
                works.append(dist.all_reduce(out[lo:hi], op=dist.ReduceOp.SUM, group=self.group, async_op=True))
        for w in works:
            w.wait()
        return out

    def _ensure_peer_buffers(self, h8: torch.Tensor) -> bool:
        """Allocates and exchanges the peer-addressable buffers on first use.  The ranks agree on the
        outcome (a MIN all-reduce of a success flag): with comm="auto" a failure anywhere -- peer
        mapping not permitted on this machine -- turns every rank to the NCCL mode; with
        comm="fused" it is an error."""
        import torch.distributed as dist
        tokens, d = h8.shape[0], self.s.w_down.shape[0]
        if self._peer is not None and self._peer.tokens == tokens and self._peer.d == d:
            return True
        err = None
        try:
            pb = PeerBuffers(tokens, d, h8.device, self.group)
        except Exception as e:  # noqa: BLE001  (whatever the allocator or the exchange raised)
            pb, err = None, e
        ok = torch.tensor([1 if pb is not None else 0], device=h8.device, dtype=torch.int32)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=self.group)
        if int(ok.item()) == 0:
            if self.comm == "fused":
                raise RuntimeError(f"comm='fused': the ranks could not map each other's memory: {err!r}")
            self._no_peer_buffers = True
            return False
        self._peer = pb
        pb.barrier()
        return True

    def _down_fused(self, h8: torch.Tensor) -> torch.Tensor:
        from . import abi
        d = self.s.w_down.shape[0]
        pb = self._peer
        # rank r's partial sums of block i (token rows [i * rows, (i + 1) * rows)) -> slot r of rank i's stage
        abi.fp8_gemm_nt(h8, self.s.w_down, torch.bfloat16, 1.0 / self.act_scale, self.s.s_down_inv, None,
                        route=(pb.stage_ptrs, pb.rows, pb.rank * pb.rows))
        if self.skip_collective:
            return pb.out
        pb.barrier()   # every rank's partial sums have landed
        abi.tp_reduce_bcast(pb.stage, pb.out_ptrs, pb.rank, pb.rows, d)
        pb.barrier()   # every rank's rows of the result have landed (and the stages are free again)
        return pb.out

    __call__ = forward


def mlp_flops(tokens: int, d_model: int, ffn: int) -> float:
    """2*T*d*f for each of gate, up and down."""
    return 3 * 2.0 * tokens * d_model * ffn
