"""OaMoE: sparse dropless top-k mixture of experts with shared experts, load-balance and z losses.

Reference: Source/Private/Oa/Ml/Nn/Moe/Moe.cpp:32-352 (structure, parameter names, forward, balancing losses,
telemetry).  Structure kept: RMSNorm -> router Linear -> softmax -> top-k on (logits + routing bias) ->
renormalised route weights over the UNBIASED probabilities -> expert-major packing -> grouped gate_up GEMM ->
SiluMul -> grouped down GEMM -> weighted combine -> shared experts added unconditionally -> x + out.
Checkpoint names: norm.weight, router.{weight,bias}, expert_gate_up_weight [E,2F,D], expert_gate_up_bias [E,2F],
expert_down_weight [E,D,F], expert_down_bias [E,D], shared_expert.<i>.{gate_up,down}.{weight,bias}, state
routing_bias [1,E].

The routed path is ONE autograd node (`_routed_experts`): router, plan, gather, two grouped tensor-core GEMMs and
the combine run as a fixed sequence of kernels with static shapes (the packed buffer has the dropless worst-case
size), so the whole layer is CUDA-graph capturable.  With an expert-parallel group (parallel/ep.py) the gather
and combine become the all-to-all dispatch / combine over peer memory.
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from ...core import fn_matrix as F
from ...core.matrix import OaMatrix
from ...ops import kernels as K
from ...ops import moe as M
from .. import autograd as AG
from ..module import OaModule
from .layers import OaLinear, OaRmsNorm


class OaMoeExpert(OaModule):
    """One always-on SwiGLU expert: down(silu(gate) * up) with a packed gate_up projection."""

    def __init__(self, d_model: int, d_ff: int, init_std: Optional[float] = None):
        super().__init__()
        self.DFF = d_ff
        self.GateUp = self.RegisterModule("gate_up", OaLinear(d_model, 2 * d_ff, True, init_std))
        self.Down = self.RegisterModule("down", OaLinear(d_ff, d_model, True, init_std))

    def Forward(self, x: OaMatrix, residual: Optional[OaMatrix] = None) -> OaMatrix:
        h = F.Swiglu(self.GateUp.Forward(x))
        return F.Linear(h, self.Down.Weight.Data, self.Down.Bias.Data, residual=residual)


def _routed_experts(x: OaMatrix, logits: OaMatrix, wgu: OaMatrix, bgu: OaMatrix, wd: OaMatrix, bd: OaMatrix, k: int,
                    sel_bias: Optional[torch.Tensor], base: Optional[OaMatrix], layer: "OaMoE") -> OaMatrix:
    F._ctx_add("MoeRouter")
    tx = F._c(x.Tensor())
    tl = F._c(logits.Tensor())
    E = tl.shape[1]
    probs, idx, w = M.router(tl, k, sel_bias)
    F._ctx_add("MoeExpertPlan")
    P = M.plan(idx, E) if layer.Dispatcher is None else None
    twgu, tbgu, twd, tbd = wgu.Tensor(), bgu.Tensor() if bgu is not None else None, wd.Tensor(), bd.Tensor() if bd is not None else None
    if layer.Dispatcher is None:
        F._ctx_add("MoeGather")
        px = M.gather(tx, P)
        F._ctx_add("GroupedLinearM")
        gu = M.grouped_linear(px, twgu, tbgu, P)
        F._ctx_add("SiluMul")
        h = K.swiglu_fwd(gu)
        F._ctx_add("GroupedLinearM")
        po = M.grouped_linear(h, twd, tbd, P)
        F._ctx_add("MoeCombine")
        out_t = M.combine(po, w, P, base.Tensor() if base is not None else None)
        saved = (P, px, gu, h, po)
    else:
        out_t, saved = layer.Dispatcher.Forward(tx, idx, w, twgu, tbgu, twd, tbd, base.Tensor() if base is not None else None)
    layer._last = (probs, idx, w, P.counts if P is not None else saved[0].counts_global)
    out = OaMatrix(out_t)

    def back(g):
        g = F._c(g)
        if layer.Dispatcher is None:
            P_, px_, gu_, h_, po_ = saved
            dpo, dw = M.combine_bwd(po_, w, P_, g)
            dh = M.grouped_linear(dpo, twd, None, P_, b_mn=True)
            dwd = _expert_grad(wd, lambda o, a: M.grouped_weight_grad(dpo, h_, P_, out=o, accumulate=a), twd)
            dbd = M.grouped_bias_grad(dpo, P_) if bd is not None and bd.RequiresGrad() else None
            dgu = K.swiglu_bwd(gu_, dh)
            dpx = M.grouped_linear(dgu, twgu, None, P_, b_mn=True)
            dwgu = _expert_grad(wgu, lambda o, a: M.grouped_weight_grad(dgu, px_, P_, out=o, accumulate=a), twgu)
            dbgu = M.grouped_bias_grad(dgu, P_) if bgu is not None and bgu.RequiresGrad() else None
            dx = M.gather_bwd(dpx, P_)
        else:
            dx, dw, dwgu, dbgu, dwd, dbd = layer.Dispatcher.Backward(saved, g, w, wgu, bgu, wd, bd)
        dlogits = M.router_bwd(probs, idx, w, dw, None, 0.0, tl.dtype)
        return (dx, dlogits, dwgu, dbgu, dwd, dbd, g if base is not None else None)

    return AG.attach("MoeRoutedExperts", out, [x, logits, wgu, bgu, wd, bd, base], back)


def _expert_grad(param: OaMatrix, compute, like: torch.Tensor):
    """Writes a stacked expert-weight gradient straight into the parameter's gradient buffer when it has one."""
    if not param.RequiresGrad():
        return None
    sink = param.GradSink() if param.IsLeaf() else None
    if sink is not None:
        compute(sink[0], sink[1])
        return None
    return compute(None, False)


class OaMoE(OaModule):
    def __init__(self, d_model: int, d_ff: int, num_experts: int, experts_per_token: int = 2, rms_eps: float = 1e-6,
                 num_shared_experts: int = 0, init_std: Optional[float] = None, expert_bias: bool = True):
        super().__init__()
        if d_model <= 0 or d_ff <= 0 or num_experts <= 0:
            raise ValueError("OaMoE dimensions and expert count must be positive")
        self.DModel, self.DFF, self.NumExperts = d_model, d_ff, num_experts
        self.ExpertsPerToken = max(1, min(experts_per_token, num_experts))
        self.Norm = self.RegisterModule("norm", OaRmsNorm(d_model, rms_eps))
        self.Router = self.RegisterModule("router", OaLinear(d_model, num_experts, True, init_std))
        gb, db = math.sqrt(1.0 / d_model), math.sqrt(1.0 / d_ff)
        gate_w = F.PhiloxUniform([num_experts, 2 * d_ff, d_model], -gb, gb) if init_std is None else F.RandN([num_experts, 2 * d_ff, d_model], std=init_std)
        down_w = F.PhiloxUniform([num_experts, d_model, d_ff], -db, db) if init_std is None else F.RandN([num_experts, d_model, d_ff], std=init_std)
        self.GateUpW = self.RegisterParameter("expert_gate_up_weight", gate_w)
        self.GateUpB = self.RegisterParameter("expert_gate_up_bias", F.Zeros([num_experts, 2 * d_ff])) if expert_bias else None
        self.DownW = self.RegisterParameter("expert_down_weight", down_w)
        self.DownB = self.RegisterParameter("expert_down_bias", F.Zeros([num_experts, d_model])) if expert_bias else None
        self.SharedExperts = []
        for s in range(max(0, num_shared_experts)):
            self.SharedExperts.append(self.RegisterModule(f"shared_expert.{s}", OaMoeExpert(d_model, d_ff, init_std)))
        self.RoutingBias = OaMatrix(torch.zeros((1, num_experts), dtype=torch.float32, device=self.Router.Weight.Tensor().device))
        self.RegisterBuffer("routing_bias", self.RoutingBias)
        self.AuxAlpha, self.ZBeta, self.BalanceGamma = 0.0, 0.0, 0.0
        self.SparseExecution = True
        self.Dispatcher = None            # set by the expert-parallel plan
        self._last = None
        self.LastAuxLoss = OaMatrix(torch.zeros(1, dtype=torch.float32, device=self.RoutingBias.Tensor().device))

    # ---- configuration (Moe.h)
    def SetAuxLossAlpha(self, a: float) -> None: self.AuxAlpha = float(a)
    def SetZLossBeta(self, b: float) -> None: self.ZBeta = float(b)
    def SetBalanceGamma(self, g: float) -> None: self.BalanceGamma = float(g)
    def SetSparseExecution(self, on: bool) -> None: self.SparseExecution = bool(on)
    def AuxLoss(self) -> OaMatrix: return self.LastAuxLoss

    # ---- forward
    def Forward(self, x: OaMatrix) -> OaMatrix:
        """x [T, D] -> x + routed experts + shared experts (pre-norm inside)."""
        normed = self.Norm.Forward(x)
        logits = self.Router.Forward(normed)
        sel_bias = self.RoutingBias.Tensor().reshape(-1) if self.BalanceGamma > 0 else None
        tn = normed.Tensor()
        # the grouped tensor-core kernels are bf16; an fp32 model on the GPU takes the dense formulation (same function)
        if self.SparseExecution and (not tn.is_cuda or tn.dtype == torch.bfloat16):
            out = _routed_experts(normed, logits, self.GateUpW.Data, self.GateUpB.Data if self.GateUpB else None, self.DownW.Data,
                                  self.DownB.Data if self.DownB else None, self.ExpertsPerToken, sel_bias, x, self)
        else:
            out = F.Add(x, self._dense_oracle(normed, logits, sel_bias))
        for se in self.SharedExperts:
            out = se.Forward(normed, residual=out)
        self.LastAuxLoss = self._aux_loss(logits)
        return out

    def _dense_oracle(self, normed: OaMatrix, logits: OaMatrix, sel_bias) -> OaMatrix:
        """Independent dense reference: every expert on every token, gated by the masked renormalised probabilities."""
        E, Kk = self.NumExperts, self.ExpertsPerToken
        probs = F.Softmax(logits)
        sel = logits if sel_bias is None else F.Add(logits, OaMatrix(sel_bias.to(logits.Tensor().dtype).reshape(1, E)))
        mask = F.TopKMask(sel, Kk)
        gate_un = F.Mul(probs, mask)
        gate = F.Div(gate_un, F.Reshape(F.Sum(gate_un, 1), [normed.Size(0), 1]))
        self._last = (probs.Tensor().float(), None, None, mask.Tensor().float().sum(0))
        acc = None
        for e in range(E):
            # slices of leaves: gradients flow back through explicit Slice nodes
            wgu = F.Reshape(F.Slice(self.GateUpW.Data, 0, e, e + 1), [2 * self.DFF, self.DModel])
            wd = F.Reshape(F.Slice(self.DownW.Data, 0, e, e + 1), [self.DModel, self.DFF])
            bgu = F.Reshape(F.Slice(self.GateUpB.Data, 0, e, e + 1), [2 * self.DFF]) if self.GateUpB else None
            bd = F.Reshape(F.Slice(self.DownB.Data, 0, e, e + 1), [self.DModel]) if self.DownB else None
            y = F.Linear(F.Swiglu(F.Linear(normed, wgu, bgu)), wd, bd)
            y = F.Mul(y, F.Slice(gate, 1, e, e + 1))
            acc = y if acc is None else F.Add(acc, y)
        return acc

    def _aux_loss(self, logits: OaMatrix) -> OaMatrix:
        """alpha * (E/K) * sum_e f_e * P_e (+ beta * mean(LSE^2)); f = dispatch fraction (constant), P = mean probability."""
        if self.AuxAlpha <= 0.0 and self.ZBeta <= 0.0 or self._last is None:
            return OaMatrix(torch.zeros(1, dtype=torch.float32, device=logits.Tensor().device))
        probs, idx, w, counts = self._last
        T, E = probs.shape
        Kk = self.ExpertsPerToken
        fe = counts.float() / T
        coef = self.AuxAlpha * E / Kk
        pe = K.col_sum(probs).float() / T
        val = (fe * pe).sum().reshape(1) * coef
        tl = logits.Tensor()
        zb = self.ZBeta
        lse = None
        if zb > 0.0:
            lse = torch.logsumexp(tl.float(), -1)
            val = val + zb * (lse * lse).mean().reshape(1)
        out = OaMatrix(val)

        def back(g):
            gs = g.reshape(1).float()
            if idx is not None:
                zeros = torch.zeros_like(w)
                dl = M.router_bwd(probs, idx, w, zeros, fe * gs, coef / T, torch.float32)
            else:
                dp = (fe * gs * coef / T).reshape(1, E).expand(T, E)
                dl = probs * (dp - (dp * probs).sum(-1, keepdim=True))
            if zb > 0.0:
                dl = dl + (2.0 * zb / T) * gs * lse[:, None] * probs
            return (dl.to(tl.dtype),)

        return AG.attach("MoeAuxLoss", out, [logits], back)

    # ---- telemetry / balancing (host side; need a prior Execute + Sync)
    def LastLoadFraction(self):
        if self._last is None:
            return []
        counts = self._last[3].float()
        return (counts / max(1.0, float(counts.sum()))).cpu().tolist()

    def UpdateRoutingBias(self) -> None:
        """Aux-loss-free balancing: bias -= gamma * sign(load - target) (MoeRoutingBiasUpdate.slang:1-29)."""
        if self.BalanceGamma <= 0 or self._last is None:
            return
        counts = self._last[3].float()
        target = counts.sum() / self.NumExperts
        self.RoutingBias.Tensor().sub_(self.BalanceGamma * torch.sign(counts - target).reshape(1, -1))
