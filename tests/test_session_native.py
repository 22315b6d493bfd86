"""Semantic graph, lowering analysis, execution session (stable frame, batch hazards) and execution plan."""
import pytest
import torch

from oa_b200.core.registry import OaOperationRegistry
from oa_b200.runtime.graph import OaAccess, OaComputeGraph
from oa_b200.runtime.session import (OaAnalyzeSemanticLowering, OaExecutionPlan, OaExecutionSession, OaSemanticGraph,
                                     OaValidateSemanticLowering)


def _mlp():
    g = OaSemanticGraph()
    x = g.AddValue("x", (8, 16), external=True)
    w = g.AddValue("w", (32, 16), external=True)
    h = g.AddValue("h", (8, 32))
    a = g.AddValue("a", (8, 32))
    s = g.AddValue("s", (), kind=1)
    lin = OaOperationRegistry.Find("Linear") or "Linear"
    op0 = g.AddOperation(lin, [x, w], [h], attributes={"epilogue": "none"})
    op1 = g.AddOperation("Gelu", [h], [a])
    op2 = g.AddOperation("Sum", [a], [s], control=[op0])
    return g, (x, w, h, a, s), (op0, op1, op2)


def test_semantic_graph_build_validate_report():
    g, (x, w, h, a, s), (op0, op1, op2) = _mlp()
    assert g.ValueCount() == 5 and g.OperationCount() == 3
    assert g.Validate().IsOk()
    v = g.FindValue(h)
    assert v.Name == "h" and v.Shape == [8, 32] and v.Producer == op0 and not v.External
    assert g.FindValue(99) is None
    rep = g.DebugReport("mlp")
    assert rep["name"] == "mlp" and len(rep["operations"]) == 3
    assert rep["operations"][0]["attributes"] == {"epilogue": "none"} and rep["values"][4]["shape"] == []
    with pytest.raises(ValueError):
        g.AddOperation("Relu", [a], [h])            # h already has a producer
    with pytest.raises(ValueError):
        g.AddOperation("Relu", [a], [x])            # external values are inputs only
    bad = OaSemanticGraph()
    p, q = bad.AddValue("p", (4,)), bad.AddValue("q", (4,))
    bad.AddOperation("Neg", [p], [q])               # p is read but nothing produces it
    st = bad.Validate()
    assert not st.IsOk() and "before it is produced" in st.message
    copy = OaSemanticGraph()
    assert not copy.CopyFrom(bad).IsOk() and copy.CopyFrom(g).IsOk() and copy.OperationCount() == 3


def test_autograd_provenance():
    g, vals, (op0, op1, op2) = _mlp()
    lin = g.Operation(op0)
    if lin.Differentiation == 0:                     # bare-name contract: not differentiable
        assert not g.AttachAutograd(op0, 0, 1).IsOk()
        return
    assert g.AttachAutograd(op0, 0, 7).IsOk() and not g.AttachAutograd(op0, 0, 7).IsOk()
    assert not g.AttachAutograd(op0, 3, 8).IsOk()
    da, dx = g.AddValue("da", (8, 32), external=True), g.AddValue("dx", (8, 16))
    b0 = g.AddOperation("LinearDataBwd", [da, vals[1]], [dx])
    assert not g.CompleteAutograd(op0, 9, b0, 1).IsOk()
    assert g.CompleteAutograd(op0, 7, b0, 1).IsOk() and not g.CompleteAutograd(op0, 7, b0, 1).IsOk()
    assert g.Operation(b0).BackwardOf == op0 and g.Operation(b0).BackwardSequence == 7 and g.Validate().IsOk()


def test_lowering_analysis():
    g, _, (op0, op1, op2) = _mlp()
    # Linear + Gelu share one launch (GEMM epilogue); Sum takes two launches; one launch outside any contract
    a = OaAnalyzeSemanticLowering(g, [[op0, op1], [op2], [op2], []])
    assert (a.SchemaOwnedNodeCount, a.CompatibilityNodeCount) == (3, 1)
    assert (a.DirectOperationCount, a.DecomposedOperationCount, a.FusedOperationCount, a.FusedNodeCount) == (0, 1, 2, 1)
    assert a.MaximumNodesPerOperation == 2 and a.MaximumOperationsPerNode == 2 and a.ExecutableNodeCounts == [1, 1, 2]
    assert OaAnalyzeSemanticLowering(g, [[op0], [op1], [op2]]).DirectOperationCount == 3
    assert not OaValidateSemanticLowering(g, [[op0], [op1]]).IsOk()          # Sum has no launch
    assert not OaValidateSemanticLowering(g, [[op0], [op1], [7]]).IsOk()     # unknown operation
    assert OaValidateSemanticLowering(g, [[op0, op1, op2]]).IsOk()


def test_stable_resource_frame():
    s = OaExecutionSession("cpu")
    ptrs = []
    for step in range(3):
        s.BeginFrame()
        a = s.Temp((64, 32), torch.float32)
        b = s.Temp((100,), torch.bfloat16)
        a.fill_(step); b.zero_()
        stable = s.EndFrame()
        ptrs.append((a.data_ptr(), b.data_ptr()))
        assert stable == (step > 0)
    assert ptrs[0] == ptrs[1] == ptrs[2] and s.SlotCount() == 2 and s.StableFrameCount() == 2
    s.BeginFrame()
    a = s.Temp((64, 32)); b = s.Temp((5000,), torch.bfloat16)      # second slot must grow
    assert not s.EndFrame() and a.data_ptr() == ptrs[0][0] and s.SlotGeneration(1) == 2 and b.numel() == 5000
    s.BeginFrame(); s.Temp((8,)); assert not s.EndFrame()           # fewer requests than before
    assert s.Trim() == 1 and s.SlotCount() == 1 and s.BytesHeld() == 64 * 32 * 4
    with pytest.raises(RuntimeError):
        s.Temp((1,))
    s.BeginFrame()
    with pytest.raises(RuntimeError):
        s.BeginFrame()


def test_batch_hazards_and_graph_reuse():
    s = OaExecutionSession()
    s.BeginAsyncBatch()
    assert s.AddToBatch([(1, 1), (2, 2)]) == []          # reads 1, writes 2
    assert s.AddToBatch([(1, 1), (3, 2)]) == []          # read-read on 1: no hazard
    assert s.AddToBatch([(2, 1), (3, 1)]) == [0, 1]      # read after write on both
    assert s.AddToBatch([(1, 2)]) == [0, 1]              # write after read
    assert s.SubmitBatch(event_id=42) == 4 and s.PendingEvent() == 42
    with pytest.raises(RuntimeError):
        s.AddToBatch([(1, 1)])
    assert not s.TakeGraph(0xabc)
    s.ParkGraph(0xabc)
    assert s.TakeGraph(0xabc) and not s.TakeGraph(0xabc) and s.ReuseStats() == (1, 2)


def test_execution_plan_matches_structure():
    def build(extra=False, kernel="gelu"):
        g = OaComputeGraph()
        g.AddNode("gemm", [(1, 1024, OaAccess.Read), (2, 1024, OaAccess.Write)])
        g.AddNode(kernel, [(2, 1024, OaAccess.ReadWrite)])
        if extra:
            g.AddNode("sum", [(2, 1024, OaAccess.Read), (3, 4, OaAccess.Write)])
        return g
    s = OaExecutionSession()
    plan = OaExecutionPlan(build(), s)
    assert plan.NodeCount() == 2 and plan.Hash() == build().Hash()
    assert plan.Matches(build()) and plan.FirstMismatch(build(kernel="relu")) == 1 and plan.FirstMismatch(build(extra=True)) == 2
    assert plan.NoteReplay() == 1 and plan.NoteReplay() == 2 and plan.ReplayCount() == 2
