"""FX graph passes that turn a PT2E quantize/dequantize graph into the FP8 operators.

A graph exported after PT2E FP8 quantisation holds, around every linear layer and batched
matmul, ``quantize_per_tensor -> dequantize_per_tensor`` pairs (namespace
``quantized_decomposed``) feeding plain ``aten.mm / addmm / bmm``.  The passes here rewrite
those patterns onto the operators this package implements:

==========================================  =====================================================
pattern                                      replacement
==========================================  =====================================================
``mm/addmm(dq(q(x)), transpose(dq(wq)))``    ``hpu.fp8_gemm_v2(q(x), False, wq, True, None, bf16,
                                             s_x, s_w, bias)``
``bmm(dq(a)…views…, dq(b)…views/T…)``        ``hpu.fp8_gemm_v2(a, False, b, trans_B, None, bf16,
                                             s_a, s_b, None, False)``
``quantize_per_tensor(x, s, …)``             ``hpu.cast_to_fp8_v2(x, 1/s, False, False, e4m3)[0]``
``view -> fp8_gemm_v2 -> view``              the leading dimensions are kept through the GEMM
==========================================  =====================================================

Same rewrites, order and entry point (``PatternMatchAndReplacer(gm).run()``) as
``python_packages/habana_frameworks/torch/core/pattern_matcher.py:98-135`` (quantize -> cast),
``:163-289`` (bmm), ``:295-412`` (mm / addmm), ``:418-486`` (views) and ``:492-511`` (driver) of
the reference.  The dequantisation scale of a tensor (``x ~ q * s``) is exactly the
``*_scale_inv`` argument of ``fp8_gemm_v2``; scales become one-element buffers of the graph
module.  Differences: a transpose that is folded into the GEMM always sets ``trans_B`` (the
reference sets it only when the node came from ``nn.Linear``), and the device of the scale
buffers is a parameter.
"""
from __future__ import annotations

import operator
from typing import List, Optional

import torch
import torch.fx as fx

_VIEW_LIKE = ("view.default", "expand.default", "clone.default", "_unsafe_view.default", "slice.Tensor", "transpose.int")
_RESHAPES = ("view.default", "_unsafe_view.default")


def _name(node) -> Optional[str]:
    if isinstance(node, fx.Node) and node.op == "call_function":
        return getattr(node.target, "__name__", None)
    return None


def _is(node, *names) -> bool:
    return _name(node) in names


def _hpu():
    import b200_hpu_ops  # noqa: F401  (registers the hpu:: operators)
    return torch.ops.hpu


class _Rewriter:
    def __init__(self, gm: fx.GraphModule, device):
        self.gm, self.g, self.device = gm, gm.graph, device
        self.replaced = 0
        self._n_buf = 0

    def scale_buffer(self, value, before: fx.Node) -> fx.Node:
        """Registers ``tensor(value)`` as a buffer and returns a get_attr node placed before `before`."""
        while True:
            name = f"_fp8_scale_{self._n_buf}"
            self._n_buf += 1
            if not hasattr(self.gm, name):
                break
        self.gm.register_buffer(name, torch.tensor(float(value), dtype=torch.float32, device=self.device))
        with self.g.inserting_before(before):
            return self.g.get_attr(name)

    def finish(self, dead: List[Optional[fx.Node]]):
        # users first: erase in reverse topological order, and only what became unused
        order = {n: i for i, n in enumerate(self.g.nodes)}
        for n in sorted({d for d in dead if d is not None}, key=lambda d: -order.get(d, -1)):
            if n in order and len(n.users) == 0:
                self.g.erase_node(n)
        self.g.lint()
        self.gm.recompile()


def _trace_to_dequant(node):
    """Walks up through shape-only nodes; returns (dequantize node or None, nodes passed)."""
    passed = []
    while isinstance(node, fx.Node) and node.op == "call_function":
        if _is(node, "dequantize_per_tensor.default"):
            return node, passed
        if _name(node) not in _VIEW_LIKE:
            break
        passed.append(node)
        node = node.args[0]
    return None, passed


def _last_two_dims(tr: fx.Node) -> bool:
    """transpose.int over the last two dimensions?  With the operand's rank known from the node's
    meta the test is exact; without it, negative indices or (1, 2) / (2, 3) are taken as such
    (the operands of a bmm are 3-D, or 4-D before the reshape that flattens batch and heads)."""
    d0, d1 = tr.args[1], tr.args[2]
    src = tr.args[0]
    meta = src.meta.get("val", src.meta.get("tensor_meta")) if isinstance(src, fx.Node) else None
    if meta is not None:
        r = len(meta.shape)
        return {d0 % r, d1 % r} == {r - 1, r - 2}
    return {d0, d1} in ({-1, -2}, {1, 2}, {2, 3})


# ----------------------------------------------------------------------------------------------
def replace_pattern_quant_dequant_mm_addmm(gm: fx.GraphModule, device="cuda") -> int:
    rw = _Rewriter(gm, device)
    hpu = _hpu()
    dead: List[Optional[fx.Node]] = []
    for node in list(gm.graph.nodes):
        if not _is(node, "mm.default", "addmm.default"):
            continue
        addmm = _is(node, "addmm.default")
        bias = node.args[0] if addmm else None
        x_arg, w_arg = (node.args[1], node.args[2]) if addmm else (node.args[0], node.args[1])
        # weight side: transpose(dequantize(wq))
        if not (_is(w_arg, "transpose.int") and _is(w_arg.args[0], "dequantize_per_tensor.default")):
            continue
        w_t, w_dq = w_arg, w_arg.args[0]
        # activation side: dequantize(q), possibly under one reshape
        x_view = x_arg if _is(x_arg, "view.default") else None
        x_dq = x_view.args[0] if x_view is not None else x_arg
        if not _is(x_dq, "dequantize_per_tensor.default"):
            continue
        x_q, w_q = x_dq.args[0], w_dq.args[0]
        if x_view is not None and len(x_view.users) == 1:
            x_view.args = (x_q,) + tuple(x_view.args[1:])  # reshape the fp8 tensor instead
            gemm_in = x_view
        elif x_view is not None:
            # the reshaped activation feeds other nodes too (several projections of one
            # activation): they keep the dequantised view, this GEMM gets a view of the fp8 tensor
            with gm.graph.inserting_before(node):
                gemm_in = gm.graph.call_function(x_view.target, (x_q,) + tuple(x_view.args[1:]))
        else:
            gemm_in = x_q
        s_x = rw.scale_buffer(x_dq.args[1], node)
        s_w = rw.scale_buffer(w_dq.args[1], node)
        with gm.graph.inserting_before(node):
            gemm = gm.graph.call_function(hpu.fp8_gemm_v2.default,
                                          (gemm_in, False, w_q, True, None, torch.bfloat16, s_x, s_w, bias))
        node.replace_all_uses_with(gemm)
        dead += [node, w_t, w_dq, x_view if x_view is not gemm_in else None, x_dq]
        rw.replaced += 1
    if rw.replaced:
        rw.finish(dead)
    return rw.replaced


def replace_pattern_quant_dequant_bmm(gm: fx.GraphModule, device="cuda") -> int:
    rw = _Rewriter(gm, device)
    hpu = _hpu()
    dead: List[Optional[fx.Node]] = []
    for node in list(gm.graph.nodes):
        if not _is(node, "bmm.default"):
            continue
        a_dq, a_path = _trace_to_dequant(node.args[0])
        b_dq, b_path = _trace_to_dequant(node.args[1])
        if a_dq is None or b_dq is None:
            continue
        # The rewrite feeds the fp8 tensors through the shape-only nodes between the dequantise
        # nodes and this bmm.  That is only right when nothing else reads those nodes: with a
        # second consumer the operand is left alone and this bmm keeps its bf16 form.
        if any(len(n.users) != 1 for n in [a_dq, b_dq] + a_path + b_path):
            continue
        # fold a transpose of the last two dims on the B side into trans_B, drop a no-op expand.
        # b_path lists the shape-only nodes from the bmm upwards, so b_path[:i] comes AFTER node i
        # in data flow and sees swapped trailing dims once the transpose is gone.
        trans_b = False
        for i, n in enumerate(b_path):
            if _is(n, "transpose.int") and len(n.users) == 1 and _last_two_dims(n):
                n.replace_all_uses_with(n.args[0])
                dead.append(n)
                trans_b = not trans_b
                for m in b_path[:i]:
                    if _name(m) in _RESHAPES or _is(m, "expand.default"):
                        shp = list(m.args[1])
                        shp[-1], shp[-2] = shp[-2], shp[-1]
                        m.args = (m.args[0], tuple(shp)) + tuple(m.args[2:])
            elif _is(n, "expand.default") and len(n.users) == 1:
                meta = n.args[0].meta.get("val", n.args[0].meta.get("tensor_meta")) if isinstance(n.args[0], fx.Node) else None
                if meta is not None and tuple(meta.shape) == tuple(n.args[1]):
                    n.replace_all_uses_with(n.args[0])
                    dead.append(n)
        s_a = rw.scale_buffer(a_dq.args[1], node)
        s_b = rw.scale_buffer(b_dq.args[1], node)
        with gm.graph.inserting_before(node):
            gemm = gm.graph.call_function(hpu.fp8_gemm_v2.default,
                                          (node.args[0], False, node.args[1], trans_b, None, torch.bfloat16, s_a, s_b, None, False))
        node.replace_all_uses_with(gemm)
        a_dq.replace_all_uses_with(a_dq.args[0])
        b_dq.replace_all_uses_with(b_dq.args[0])
        dead += [node, a_dq, b_dq]
        rw.replaced += 1
    if rw.replaced:
        rw.finish(dead)
    return rw.replaced


def replace_quantize_with_cast(gm: fx.GraphModule, fp8_dtype=torch.float8_e4m3fn) -> int:
    hpu = _hpu()
    n_done = 0
    for node in list(gm.graph.nodes):
        if not _is(node, "quantize_per_tensor.default"):
            continue
        scale = node.args[1]
        with gm.graph.inserting_before(node):
            if isinstance(scale, fx.Node):
                inv = gm.graph.call_function(torch.ops.aten.reciprocal.default, (scale,))
                cast = gm.graph.call_function(hpu.cast_to_fp8_v2.default, (node.args[0], inv, False, False, fp8_dtype))
            else:
                cast = gm.graph.call_function(hpu.cast_to_fp8_v2.scalar, (node.args[0], 1.0 / float(scale), False, False, fp8_dtype))
            out = gm.graph.call_function(operator.getitem, (cast, 0))
        node.replace_all_uses_with(out)
        gm.graph.erase_node(node)
        n_done += 1
    if n_done:
        gm.graph.lint()
        gm.recompile()
    return n_done


def replace_pattern_view_mm_view(gm: fx.GraphModule) -> int:
    """``view([B*S, K]) -> fp8_gemm_v2 -> view([B, S, N])``: let the GEMM see ``[B, S, K]`` (its
    output shape follows torch.matmul) and drop the output reshape."""
    n_done = 0
    for node in list(gm.graph.nodes):
        if _name(node) not in ("fp8_gemm_v2", "fp8_gemm_v2.default") or len(node.users) != 1:
            continue
        vin, vout = node.args[0], next(iter(node.users))
        if not (_name(vin) in _RESHAPES and len(vin.users) == 1 and _name(vout) in _RESHAPES):
            continue
        in_shape, out_shape = list(vin.args[1]), list(vout.args[1])
        if len(out_shape) < 3 or len(in_shape) > len(out_shape):
            continue
        vin.args = (vin.args[0], tuple(out_shape[:-1] + [in_shape[-1]])) + tuple(vin.args[2:])
        vout.replace_all_uses_with(node)
        gm.graph.erase_node(vout)
        n_done += 1
    if n_done:
        gm.graph.lint()
        gm.recompile()
    return n_done


class PatternMatchAndReplacer:
    """Runs the passes in the reference's order; ``replaced`` counts the rewrites of each."""

    def __init__(self, graph_module: fx.GraphModule, device="cuda"):
        self._gm, self._device = graph_module, device
        self.replaced = {}

    def run(self):
        self.replaced["mm_addmm"] = replace_pattern_quant_dequant_mm_addmm(self._gm, self._device)
        self.replaced["bmm"] = replace_pattern_quant_dequant_bmm(self._gm, self._device)
        self.replaced["quantize"] = replace_quantize_with_cast(self._gm)
        self.replaced["views"] = replace_pattern_view_mm_view(self._gm)
        return self._gm
