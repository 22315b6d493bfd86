"""Which fused engines a Transformer block runs with, decided by the native fusion planner
(csrc/runtime/dnn.cpp; reference: Source/Public/Oa/Runtime/Dnn.h:16-100, whose OaDnnPlanner partitions a layer's operation
graph into Portable / BlasLtEpilogue / PackedQkv / GatedFfn / ResidualNorm / FlashAttention / GroupedMoe engines).

A block describes itself as an operation graph (norm, the three projections, attention, output projection, residual add,
the FFN of its kind), the planner partitions it, and the layer code of `ml/nn/layers.py` takes the fused call for every
engine the plan holds and the composition of plain operations otherwise.  `OA_DNN_DISABLE=PackedQkv,GatedFfn,...` (engine
names, or `all`) removes engines from every plan: the differential switch between the fused and the portable lowering
of the same block.  Plans are cached per block description.
"""
from __future__ import annotations

import os
from dataclasses import dataclass, field
from typing import Dict, List, Tuple

from ...runtime.graph import OaDnnEngineType, OaDnnGraph, OaDnnOpType, OaDnnPlanner


@dataclass
class OaBlockPlan:
    PackedQkv: bool = False
    FlashAttention: bool = False
    GatedFfn: bool = False
    GemmEpilogue: bool = False
    ResidualNorm: bool = False
    GraphHash: int = 0
    Engines: List[str] = field(default_factory=list)      # engine of every partition, in plan order
    Disabled: Tuple[str, ...] = ()


_cache: Dict[tuple, OaBlockPlan] = {}


def DisabledEngines() -> Tuple[str, ...]:
    raw = os.environ.get("OA_DNN_DISABLE", "").strip()
    if not raw:
        return ()
    names = {e.name for e in OaDnnEngineType}
    if raw.lower() == "all":
        return tuple(sorted(names - {"Portable"}))
    out = []
    for n in raw.split(","):
        n = n.strip()
        if n not in names:
            raise ValueError(f"OA_DNN_DISABLE: unknown engine {n!r} (known: {', '.join(sorted(names))})")
        out.append(n)
    return tuple(sorted(out))


def PlanTransformerBlock(d_model: int, d_ff: int, ffn_kind: str, bias: bool, flash_ok: bool, rows: int = 128,
                         training: bool = True) -> OaBlockPlan:
    """`ffn_kind`: "gelu" (Linear + bias + GELU, Linear), "swiglu" (gate / up / down) or "moe" (the FFN is not planned here)."""
    disabled = DisabledEngines()
    key = (d_model, d_ff, ffn_kind, bool(bias), bool(flash_ok), bool(training), disabled)
    hit = _cache.get(key)
    if hit is not None:
        return hit
    g = OaDnnGraph()
    T = OaDnnOpType
    ids = iter(range(1, 1000))
    D, Fd = d_model, d_ff

    def mat(shape, external=False) -> int:
        i = next(ids)
        st = g.AddMatrix(i, shape, 1, external)
        assert st.IsOk(), st.message
        return i

    def op(t, ins, outs) -> None:
        st = g.AddOp(t, ins, outs, training)
        assert st.IsOk(), st.message

    def linear(x, w_shape, out_cols, with_bias) -> int:
        w = mat(w_shape, True)
        y = mat([rows, out_cols])
        op(T.Matmul, [x, w], [y])
        if with_bias:
            b, yb = mat([out_cols], True), mat([rows, out_cols])
            op(T.BiasAdd, [y, b], [yb])
            return yb
        return y

    x = mat([rows, D], True)
    nw = mat([D], True)
    h = mat([rows, D])
    op(T.RmsNorm, [x, nw], [h])
    q, k, v = (linear(h, [D, D], D, bias) for _ in range(3))
    a = mat([rows, D])
    if flash_ok:
        op(T.FlashAttentionCausal, [q, k, v], [a])
    else:                                   # materialised attention: scores, probabilities, values as plain products
        s = mat([rows, rows])
        op(T.Matmul, [q, k], [s])
        op(T.Matmul, [s, v], [a])
    o = linear(a, [D, D], D, bias)
    x1 = mat([rows, D])
    op(T.Add, [x, o], [x1])
    if ffn_kind != "moe":
        nw2 = mat([D], True)
        h2 = mat([rows, D])
        op(T.RmsNorm, [x1, nw2], [h2])
        if ffn_kind == "gelu":
            z = linear(h2, [Fd, D], Fd, True)
            zg = mat([rows, Fd])
            op(T.Gelu, [z], [zg])
            f = linear(zg, [D, Fd], D, bias)
        else:
            gate, up = linear(h2, [Fd, D], Fd, False), linear(h2, [Fd, D], Fd, False)
            sg, gu = mat([rows, Fd]), mat([rows, Fd])
            op(T.Silu, [gate], [sg])
            op(T.Multiply, [sg, up], [gu])
            f = linear(gu, [D, Fd], D, False)
        x2 = mat([rows, D])
        op(T.Add, [x1, f], [x2])
    plan, st = OaDnnPlanner.Plan(g, allow_recompute=True)
    if plan is None:
        raise RuntimeError(f"fusion planner rejected the block graph: {st.message}")
    engines = [p.Engine.name for p in plan.Partitions]
    have = set(engines) - set(disabled)
    out = OaBlockPlan(PackedQkv="PackedQkv" in have, FlashAttention="FlashAttention" in have, GatedFfn="GatedFfn" in have,
                      GemmEpilogue="BlasLtEpilogue" in have, ResidualNorm="ResidualNorm" in have, GraphHash=plan.GraphHash,
                      Engines=engines, Disabled=disabled)
    _cache[key] = out
    return out


def ClearPlanCache() -> None:
    _cache.clear()
