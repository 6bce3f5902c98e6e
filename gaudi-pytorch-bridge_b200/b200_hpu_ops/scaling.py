"""FP8 scale management on the device: current scaling and delayed scaling.

The reference derives the scale of an FP8 tensor from its amax with ATen ops on the device
(``habana_kernels/lazy_optimizer_kernels.cpp:113-126``: ``2 ** floor(log2(fp8_max / amax))``,
kept when the amax is 0) and passes it to ``cast_to_fp8_v2`` as a one-element tensor.  The
classes here do the same with this package's kernels; no step reads a value back to the host,
so everything can be enqueued ahead (and captured in a CUDA graph).

* ``current_scaling_cast``  amax pass, scale, cast: 5 bytes per bf16 element instead of 3.
* ``DelayedScaling``        the cast uses the scale derived from EARLIER amax values (one pass,
                            3 bytes per element; the cast returns this step's amax as a
                            by-product), then the amax history ring and the scale are updated
                            for the next step.
"""
from __future__ import annotations

import torch

FP8_MAX = {torch.float8_e4m3fn: 448.0, torch.float8_e5m2: 57344.0}


def current_scaling_cast(x: torch.Tensor, dtype: torch.dtype = torch.float8_e4m3fn, stochastic_rounding: bool = False,
                         pow2: bool = True, margin: int = 0, scale: torch.Tensor | None = None, group=None, ops=None):
    """Returns (fp8 tensor, scale, amax); ``scale`` (one-element fp32, updated in place when given)
    multiplies the input, its reciprocal is the ``scale_inv`` of the consumer.

    ``group``: the tensor is a shard of a larger one (rows of an activation split over the
    ranks of a process group): the amax is made global with one 4-byte MAX all-reduce before
    the scale is derived, so that every rank casts with the same scale and the shards
    concatenate to the bytes of the unsharded cast.  Nothing else crosses the ranks.
    ``ops``: operator namespaces ``(b200q-like, hpu-like)``; the default is this package's CUDA
    operators (CPU ranks in tests pass stand-ins)."""
    b200q, hpu = ops if ops is not None else (torch.ops.b200q, torch.ops.hpu)
    amax = b200q.amax(x)
    if group is not None:
        import torch.distributed as dist
        dist.all_reduce(amax, op=dist.ReduceOp.MAX, group=group)
    if scale is None:
        scale = torch.ones(1, dtype=torch.float32, device=x.device)
    b200q.scale_from_amax_(scale, amax, FP8_MAX[dtype], pow2, margin)
    out, _ = hpu.cast_to_fp8_v2(x, scale, stochastic_rounding, False, dtype, [1])
    return out, scale, amax


class DelayedScaling:
    """amax-history scaling for one tensor role (activations of a layer, a weight, ...)."""

    def __init__(self, device, dtype: torch.dtype = torch.float8_e4m3fn, history_len: int = 16, use_max: bool = True,
                 pow2: bool = True, margin: int = 0):
        self.dtype = dtype
        self.fp8_max = FP8_MAX[dtype]
        self.history = torch.zeros(history_len, dtype=torch.float32, device=device)
        self.scale = torch.ones(1, dtype=torch.float32, device=device)
        self.pos = 0
        self.use_max, self.pow2, self.margin = use_max, pow2, margin

    def cast(self, x: torch.Tensor, stochastic_rounding: bool = False) -> torch.Tensor:
        # the cast must see the scale of the earlier steps: clone it before the update below
        # overwrites it on the same stream (stream order makes the clone safe)
        scale_now = self.scale.clone()
        out, amax = torch.ops.hpu.cast_to_fp8_v2(x, scale_now, stochastic_rounding, True, self.dtype, [1])
        torch.ops.b200q.amax_history_update_(self.scale, self.history, self.pos, amax, self.use_max, self.fp8_max,
                                             self.pow2, self.margin)
        self.pos = (self.pos + 1) % self.history.numel()
        self.last_scale = scale_now
        return out
