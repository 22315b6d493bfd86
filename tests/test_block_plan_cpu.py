"""The fusion planner chooses the engines of a Transformer block (Runtime/Dnn.h:16-100 of the reference: OaDnnPlanner
partitions a layer's operation graph into fused engines); the layer code runs the fused call for every engine in the plan
and the composition of plain operations otherwise.  Both lowerings are the same function."""
import pytest
import torch

from oa_b200.core import fn_matrix as F
from oa_b200.ml.autograd import OaGradientTape
from oa_b200.ml.nn import block_plan as BP
from oa_b200.ml.nn.layers import OaTransformerBlock
from oa_b200.runtime.engine import OaContext


def test_plans_of_the_three_block_kinds():
    BP.ClearPlanCache()
    g = BP.PlanTransformerBlock(64, 256, "gelu", True, True)
    assert g.PackedQkv and g.FlashAttention and g.GemmEpilogue and g.ResidualNorm and not g.GatedFfn
    s = BP.PlanTransformerBlock(64, 256, "swiglu", False, True)
    assert s.PackedQkv and s.GatedFfn and s.FlashAttention
    m = BP.PlanTransformerBlock(64, 0, "moe", True, False)
    assert m.PackedQkv and not m.FlashAttention and not m.GatedFfn
    assert g.GraphHash != s.GraphHash != m.GraphHash
    assert BP.PlanTransformerBlock(64, 256, "gelu", True, True) is g          # cached


def test_disable_switch(monkeypatch):
    BP.ClearPlanCache()
    monkeypatch.setenv("OA_DNN_DISABLE", "PackedQkv,GatedFfn")
    p = BP.PlanTransformerBlock(64, 256, "swiglu", False, True)
    assert not p.PackedQkv and not p.GatedFfn and p.FlashAttention and "PackedQkv" in p.Engines
    monkeypatch.setenv("OA_DNN_DISABLE", "all")
    p = BP.PlanTransformerBlock(64, 256, "gelu", True, True)
    assert not (p.PackedQkv or p.FlashAttention or p.GemmEpilogue or p.ResidualNorm)
    monkeypatch.setenv("OA_DNN_DISABLE", "Turbo")
    with pytest.raises(ValueError, match="unknown engine"):
        BP.PlanTransformerBlock(32, 64, "gelu", True, True)


def _run(kind: str, names: list):
    F.SetRngSeed(5)
    blk = OaTransformerBlock(32, 64, 8, 4, ffn=kind, norm="rms" if kind == "swiglu" else "layer", bias=kind == "gelu")
    torch.manual_seed(1)
    x = F.FromTensor(torch.randn(16, 32)).SetRequiresGrad(True)
    ctx = OaContext.GetDefault()
    ctx.BeginCollect()
    with OaGradientTape() as tape:
        y = blk.Forward(x, 2, 8)
        tape.Backward(F.Sum(F.Mul(y, y)))
    nodes, _ = ctx.EndCollect()
    names.extend(n[0] for n in nodes)
    grads = [p.Data.GradTensor().clone() for p in blk.AllParameterPtrs()]
    return y.Tensor().clone(), x.GradTensor().clone(), grads


@pytest.mark.parametrize("kind", ["gelu", "swiglu"])
def test_fused_and_portable_lowerings_agree(kind, monkeypatch):
    BP.ClearPlanCache()
    fused_names, plain_names = [], []
    y0, dx0, g0 = _run(kind, fused_names)
    monkeypatch.setenv("OA_DNN_DISABLE", "all")
    BP.ClearPlanCache()
    y1, dx1, g1 = _run(kind, plain_names)
    assert torch.allclose(y0, y1, rtol=1e-5, atol=1e-6)
    assert torch.allclose(dx0, dx1, rtol=1e-4, atol=1e-5)
    for a, b in zip(g0, g1):
        assert torch.allclose(a, b, rtol=1e-4, atol=1e-5)
    assert any("PackedLinear3" in n for n in fused_names) and not any("PackedLinear3" in n for n in plain_names)
    assert sum(n == "Linear" for n in plain_names) > sum(n == "Linear" for n in fused_names)
