"""The PT2E graph passes (b200_hpu_ops/fx_passes.py) against hand-built graphs of the shapes the
reference's passes match (python_packages/habana_frameworks/torch/core/pattern_matcher.py):
structure and fake-tensor shapes on CPU, numerics on the GPU against the oracle."""
import operator

import pytest
import torch
import torch.fx as fx
import torch.ao.quantization.fx._decomposed  # noqa: F401  (registers quantized_decomposed::*)

from oracle import hpu_oracle as O

E4M3 = torch.float8_e4m3fn
aten, qd = torch.ops.aten, torch.ops.quantized_decomposed
SX, SW = 0.02, 0.004


def _qdq(g, x, s):
    q = g.call_function(qd.quantize_per_tensor.default, (x, s, 0, -448, 448, E4M3))
    return q, g.call_function(qd.dequantize_per_tensor.default, (q, s, 0, -448, 448, E4M3))


def linear_graph(with_bias, with_views):
    """x [B,S,K] -> (view [B*S,K]) -> q/dq -> addmm/mm with transpose(dq(q(w))) -> (view [B,S,N])."""
    g = fx.Graph()
    x, w = g.placeholder("x"), g.placeholder("w")
    b = g.placeholder("b") if with_bias else None
    _, xd = _qdq(g, x, SX)
    _, wd = _qdq(g, w, SW)
    wt = g.call_function(aten.transpose.int, (wd, 0, 1))
    xin = g.call_function(aten.view.default, (xd, (6, 64))) if with_views else xd
    mm = g.call_function(aten.addmm.default, (b, xin, wt)) if with_bias else g.call_function(aten.mm.default, (xin, wt))
    out = g.call_function(aten._unsafe_view.default, (mm, (2, 3, 32))) if with_views else mm
    g.output(out)
    return fx.GraphModule(torch.nn.Module(), g)


def bmm_graph():
    """a [4,8,64], b [4,16,64]: bmm(dq(q(a)), transpose(dq(q(b)), 1, 2)) -> [4,8,16]."""
    g = fx.Graph()
    a, b = g.placeholder("a"), g.placeholder("b")
    _, ad = _qdq(g, a, SX)
    _, bd = _qdq(g, b, SW)
    bt = g.call_function(aten.transpose.int, (bd, 1, 2))
    g.output(g.call_function(aten.bmm.default, (ad, bt)))
    return fx.GraphModule(torch.nn.Module(), g)


def _names(gm):
    return [getattr(n.target, "__name__", str(n.target)) for n in gm.graph.nodes if n.op == "call_function"]


@pytest.mark.parametrize("with_bias", [False, True])
@pytest.mark.parametrize("with_views", [False, True])
def test_linear_rewrite_structure_and_meta_shapes(with_bias, with_views):
    from b200_hpu_ops.fx_passes import PatternMatchAndReplacer

    gm = linear_graph(with_bias, with_views)
    pm = PatternMatchAndReplacer(gm, device="meta")
    pm.run()
    names = _names(gm)
    assert pm.replaced["mm_addmm"] == 1 and pm.replaced["quantize"] == 2
    assert not any(n.startswith(("dequantize_per_tensor", "quantize_per_tensor", "mm.", "addmm.", "transpose")) for n in names), names
    assert names.count("fp8_gemm_v2.default") == 1 and sum(n.startswith("cast_to_fp8_v2") for n in names) == 2
    gemm = next(n for n in gm.graph.nodes if getattr(n.target, "__name__", "") == "fp8_gemm_v2.default")
    assert gemm.args[1] is False and gemm.args[3] is True and gemm.args[5] == torch.bfloat16
    assert (gemm.args[8] is None) == (not with_bias)
    if with_views:
        assert pm.replaced["views"] == 1 and "_unsafe_view.default" not in names
    # fake-tensor run through the Meta kernels
    x = torch.empty((2, 3, 64) if with_views else (6, 64), device="meta", dtype=torch.bfloat16)
    w = torch.empty(32, 64, device="meta", dtype=torch.bfloat16)
    args = (x, w) + ((torch.empty(32, device="meta", dtype=torch.bfloat16),) if with_bias else ())
    out = gm(*args)
    assert out.dtype == torch.bfloat16 and tuple(out.shape) == ((2, 3, 32) if with_views else (6, 32))


def test_bmm_rewrite_structure():
    from b200_hpu_ops.fx_passes import PatternMatchAndReplacer

    gm = bmm_graph()
    pm = PatternMatchAndReplacer(gm, device="meta")
    pm.run()
    names = _names(gm)
    assert pm.replaced["bmm"] == 1 and pm.replaced["quantize"] == 2
    assert not any(n.startswith(("dequantize", "quantize_per", "bmm", "transpose")) for n in names), names
    gemm = next(n for n in gm.graph.nodes if getattr(n.target, "__name__", "") == "fp8_gemm_v2.default")
    assert gemm.args[3] is True
    out = gm(torch.empty(4, 8, 64, device="meta", dtype=torch.bfloat16), torch.empty(4, 16, 64, device="meta", dtype=torch.bfloat16))
    assert tuple(out.shape) == (4, 8, 16) and out.dtype == torch.bfloat16


def test_untouched_when_no_pattern():
    from b200_hpu_ops.fx_passes import PatternMatchAndReplacer

    g = fx.Graph()
    x, w = g.placeholder("x"), g.placeholder("w")
    g.output(g.call_function(aten.mm.default, (x, w)))
    gm = fx.GraphModule(torch.nn.Module(), g)
    pm = PatternMatchAndReplacer(gm, device="meta")
    pm.run()
    assert sum(pm.replaced.values()) == 0 and _names(gm) == ["mm.default"]


def test_two_projections_share_one_reshaped_activation():
    """Two linears on one view of one dequantised activation (what CSE leaves of q/k/v
    projections): both must become FP8 GEMMs fed by fp8 tensors, none may be left as an aten.mm
    reading an fp8 tensor."""
    from b200_hpu_ops.fx_passes import PatternMatchAndReplacer

    g = fx.Graph()
    x, w1, w2 = g.placeholder("x"), g.placeholder("w1"), g.placeholder("w2")
    _, xd = _qdq(g, x, SX)
    xin = g.call_function(aten.view.default, (xd, (6, 64)))
    outs = []
    for w in (w1, w2):
        _, wd = _qdq(g, w, SW)
        outs.append(g.call_function(aten.mm.default, (xin, g.call_function(aten.transpose.int, (wd, 0, 1)))))
    g.output(tuple(outs))
    gm = fx.GraphModule(torch.nn.Module(), g)
    pm = PatternMatchAndReplacer(gm, device="meta")
    pm.run()
    names = _names(gm)
    assert pm.replaced["mm_addmm"] == 2 and names.count("fp8_gemm_v2.default") == 2
    assert not any(n.startswith(("mm.", "dequantize_per_tensor")) for n in names), names
    a, b = gm(torch.empty(2, 3, 64, device="meta", dtype=torch.bfloat16), torch.empty(32, 64, device="meta", dtype=torch.bfloat16),
              torch.empty(16, 64, device="meta", dtype=torch.bfloat16))
    assert tuple(a.shape) == (6, 32) and tuple(b.shape) == (6, 16)


def test_bmm_operand_with_a_second_consumer_is_left_alone():
    """A dequantised operand that something else reads as well must keep its bf16 values: the bmm
    is not rewritten rather than handing fp8 bytes to the other consumer."""
    from b200_hpu_ops.fx_passes import replace_pattern_quant_dequant_bmm

    g = fx.Graph()
    a, b = g.placeholder("a"), g.placeholder("b")
    _, ad = _qdq(g, a, SX)
    _, bd = _qdq(g, b, SW)
    bt = g.call_function(aten.transpose.int, (bd, 1, 2))
    bmm = g.call_function(aten.bmm.default, (ad, bt))
    other = g.call_function(aten.sum.default, (ad,))
    g.output((bmm, other))
    gm = fx.GraphModule(torch.nn.Module(), g)
    assert replace_pattern_quant_dequant_bmm(gm, device="meta") == 0
    assert "bmm.default" in _names(gm) and _names(gm).count("dequantize_per_tensor.default") == 2


@pytest.mark.gpu
@pytest.mark.parametrize("with_bias", [False, True])
def test_linear_rewrite_numerics(with_bias):
    from b200_hpu_ops.fx_passes import PatternMatchAndReplacer

    gm = linear_graph(with_bias, True)
    PatternMatchAndReplacer(gm, device="cuda").run()
    g = torch.Generator().manual_seed(2)
    x = torch.randn(2, 3, 64, generator=g).to(torch.bfloat16)
    w = (torch.randn(32, 64, generator=g) * 0.2).to(torch.bfloat16)
    b = torch.randn(32, generator=g).to(torch.bfloat16)
    args = (x.cuda(), w.cuda()) + ((b.cuda(),) if with_bias else ())
    out = gm(*args).cpu()
    x8, _ = O.cast_to_fp8_v2(x, 1.0 / SX, False, False, E4M3)
    w8, _ = O.cast_to_fp8_v2(w, 1.0 / SW, False, False, E4M3)
    want = O.fp8_gemm_v2(x8, False, w8, True, None, torch.bfloat16, torch.tensor(SX), torch.tensor(SW), b if with_bias else None)
    assert tuple(out.shape) == (2, 3, 32)
    assert O.rel_frobenius(out, want) <= 1e-2


@pytest.mark.gpu
def test_bmm_rewrite_numerics():
    from b200_hpu_ops.fx_passes import PatternMatchAndReplacer

    gm = bmm_graph()
    PatternMatchAndReplacer(gm, device="cuda").run()
    g = torch.Generator().manual_seed(4)
    a = torch.randn(4, 8, 64, generator=g).to(torch.bfloat16)
    b = (torch.randn(4, 16, 64, generator=g) * 0.2).to(torch.bfloat16)
    out = gm(a.cuda(), b.cuda()).cpu()
    a8, _ = O.cast_to_fp8_v2(a, 1.0 / SX, False, False, E4M3)
    b8, _ = O.cast_to_fp8_v2(b, 1.0 / SW, False, False, E4M3)
    want = O.fp8_gemm_v2(a8, False, b8, True, None, torch.bfloat16, torch.tensor(SX), torch.tensor(SW), None)
    assert O.rel_frobenius(out, want) <= 1e-2
