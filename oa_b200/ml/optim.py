"""Optimizers: OaSGD, OaAdam, OaAdamW, OaMuon, OaOptimizerComposite, OaOptimizerNoOp.

Reference: Source/Public/Oa/Ml/Optim.h:14-274, Source/Private/Oa/Ml/Optim/{AdamW,Adam,Sgd,Muon,MuonRef,OptimComposite}.cpp.

B200 design: at construction the optimizer moves its parameters into ONE flat arena per dtype (parameters become
views; rows stay 16-byte aligned) with a matching flat gradient arena, so that
  * a step is a single fused kernel over the arena (fp32 master weights for bf16 parameters, bf16 write-back),
  * weight-gradient GEMMs write straight into their slice of the gradient arena,
  * the data-parallel layer can reduce-scatter / all-gather contiguous shards (parallel/dp.py).
Hyper-parameters and the step counter live in a device buffer, so a captured training step replays correctly
(the reference's AdamWStepGraph / AdamWAdvanceGraphState idea, Source/Public/Oa/Ml/FnOptim.h:25-53).
Checkpoints store AdamM / AdamV flat in parameter order; fp32 masters are NOT stored, they are re-seeded from
the (possibly bf16) weights on load, as the reference does (Optim/AdamW.cpp:217-251).
"""
from __future__ import annotations

import math
from typing import Optional, Sequence

import numpy as np
import torch

from ..core.types import OaStatus, OaStatusCode
from ..io.oam import OamModel, OamOptimizerState
from ..ops import kernels as K
from ..runtime import engine as RT
from .module import OaParameter

_ALIGN_ELEMS = 64   # every parameter starts on a 128-byte (bf16) / 256-byte (fp32) boundary


class _Arena:
    """Flat storage for a list of parameters of one dtype, plus gradients and optimizer state."""

    def __init__(self, params: Sequence[OaParameter], allocator=None):
        self.params = list(params)
        self.dtype = params[0].Tensor().dtype
        self.device = params[0].Tensor().device
        # Placement: parameters that are views of one storage (the row slices of a packed QKV / gate-up tensor) are laid
        # out next to each other, in their order inside that storage, at the place of the group's first member, so that the
        # packed view survives the move into the arena even when other parameters (biases) were registered in between.
        # `params` / `offsets` stay in registration order: checkpoints and shards do not depend on the placement.
        first, keys = {}, []
        for i, p in enumerate(params):
            t = p.Tensor()
            sp = t.untyped_storage().data_ptr()
            first.setdefault(sp, i)
            keys.append((first[sp], t.storage_offset(), i))
        self.offsets, off = [0] * len(params), 0
        for _, _, i in sorted(keys):
            self.offsets[i] = off
            off += (params[i].NumElements() + _ALIGN_ELEMS - 1) // _ALIGN_ELEMS * _ALIGN_ELEMS
        self.numel = max(off, _ALIGN_ELEMS)
        alloc = allocator or (lambda n, dt: torch.zeros(n, dtype=dt, device=self.device))
        self.flat = alloc(self.numel, self.dtype)
        self.grad = alloc(self.numel, self.dtype)
        for p, o in zip(params, self.offsets):
            n = p.NumElements()
            view = self.flat[o:o + n].view(p.Tensor().shape)
            view.copy_(p.Tensor())
            p.Data._t = view
            p.Data.SetGradBuffer(self.grad[o:o + n].view(view.shape))
        self.master: Optional[torch.Tensor] = None

    def ensure_master(self) -> None:
        if self.dtype == torch.bfloat16 and self.master is None:
            self.master = self.flat.float()

    def reseed_master(self) -> None:
        if self.master is not None:
            self.master.copy_(self.flat)

    def gather(self, flat_state: torch.Tensor) -> np.ndarray:
        """Per-parameter slices of a flat fp32 state tensor, concatenated without the alignment padding."""
        host = flat_state.detach().float().cpu()
        return np.concatenate([host[o:o + p.NumElements()].numpy() for p, o in zip(self.params, self.offsets)]) \
            if self.params else np.zeros(0, np.float32)

    def scatter(self, flat_state: torch.Tensor, values: np.ndarray, start: int) -> int:
        host = torch.zeros(self.numel, dtype=torch.float32)
        for p, o in zip(self.params, self.offsets):
            n = p.NumElements()
            host[o:o + n] = torch.from_numpy(values[start:start + n].copy())
            start += n
        flat_state.copy_(host.to(flat_state.device))
        return start

    def unpadded(self) -> int:
        return sum(p.NumElements() for p in self.params)


class OaOptimizer:
    TypeName = "SGD"

    def __init__(self, params, lr: float):
        self.Params_ = [p for p in params if p is not None and p.RequiresGrad]
        self.Lr_ = float(lr)
        self.Step_ = 0
        self._arenas: list[_Arena] = []
        self._allocator = None
        self._built = False

    # ---- arena construction (lazy so that a parallel plan may install its allocator first)
    def SetArenaAllocator(self, fn) -> None:
        if self._built:
            raise RuntimeError("arena already built")
        self._allocator = fn

    def _build(self) -> None:
        if self._built:
            return
        self._built = True
        groups: dict = {}
        for p in self.Params_:
            groups.setdefault((p.Tensor().dtype, p.Tensor().device), []).append(p)
        self._arenas = [_Arena(ps, self._allocator) for ps in groups.values()]
        self._init_state()

    def _init_state(self) -> None:
        pass

    def Arenas(self) -> list:
        self._build()
        return self._arenas

    # ---- API
    def Step(self) -> None:
        raise NotImplementedError

    def DescribeStep(self, graph=None, engine=None) -> None:
        self.Step()

    def ZeroGrad(self) -> None:
        self._build()
        for a in self._arenas:
            RT.OaContext.GetDefault().Add("MultiFill")
            K.fill_(a.grad, 0.0)
            for p in a.params:
                p.Data._mark_grad_fresh()

    def SetLr(self, lr: float) -> None:
        self.Lr_ = float(lr)

    def Lr(self) -> float:
        return self.Lr_

    GetLr = Lr

    def GetStep(self) -> int:
        return self.Step_

    StepCount = GetStep

    def ReduceMetric(self, value: float) -> float:
        """A host scalar as every rank should see it.  One process: the value itself; a data-parallel wrapper replaces
        this with the mean over its ranks so that metric-driven decisions (save the best model) agree everywhere."""
        return float(value)

    def IsPrimaryWriter(self) -> bool:
        """Whether this process writes checkpoint files (rank 0 under data parallelism)."""
        return True

    def NotifyProgramReplay(self, count: int = 1) -> None:
        self.Step_ += count

    def SaveTo(self, oam: OamModel) -> OaStatus:
        return OaStatus.Ok()

    def ValidateLoad(self, oam: OamModel) -> OaStatus:
        return OaStatus.Ok()

    def LoadFrom(self, oam: OamModel) -> OaStatus:
        return OaStatus.Ok()

    # ---- helpers shared by the Adam family
    def _num_unpadded(self) -> int:
        return sum(a.unpadded() for a in self.Arenas())

    def _validate_counts(self, oam: OamModel, type_names, need_v: bool) -> OaStatus:
        if not oam.HasOptimizer():
            return OaStatus.Error(OaStatusCode.NotFound, "checkpoint has no optimizer section")
        st = oam.GetOptimizer()
        if st.Type not in type_names:
            return OaStatus.Error(OaStatusCode.InvalidArgument, f"optimizer type mismatch: file has {st.Type}")
        n = self._num_unpadded()
        if st.AdamM.size != n or (need_v and st.AdamV.size != n):
            return OaStatus.Error(OaStatusCode.InvalidArgument,
                                  f"optimizer state size mismatch: file {st.AdamM.size}/{st.AdamV.size}, model {n}")
        return OaStatus.Ok()


class OaOptimizerNoOp(OaOptimizer):
    def __init__(self):
        super().__init__([], 0.0)

    def Step(self) -> None:
        pass

    def ZeroGrad(self) -> None:
        pass

    def NotifyProgramReplay(self, count: int = 1) -> None:
        pass


class _AdamBase(OaOptimizer):
    Decoupled = False

    def __init__(self, params, lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.0):
        super().__init__(params, lr)
        self.Beta1_, self.Beta2_, self.Eps_, self.WeightDecay_ = float(beta1), float(beta2), float(eps), float(weight_decay)
        self.GradScale_ = 1.0
        self._clip_norm: Optional[float] = None
        self._state: Optional[torch.Tensor] = None
        self._m: list[torch.Tensor] = []
        self._v: list[torch.Tensor] = []
        self._clip_buf = None

    def _init_state(self) -> None:
        dev = self._arenas[0].device if self._arenas else RT.get_engine().Device()
        self._state = torch.tensor([float(self.Step_), self.Lr_, self.Beta1_, self.Beta2_, self.Eps_, self.WeightDecay_,
                                    self.GradScale_, 0.0], dtype=torch.float32, device=dev)
        self._m = [torch.zeros(a.numel, dtype=torch.float32, device=a.device) for a in self._arenas]
        self._v = [torch.zeros(a.numel, dtype=torch.float32, device=a.device) for a in self._arenas]
        for a in self._arenas:
            a.ensure_master()
        self._clip_buf = torch.zeros(2, dtype=torch.float32, device=dev)

    def StateBuffer(self) -> torch.Tensor:
        self._build()
        return self._state

    def SetLr(self, lr: float) -> None:
        self.Lr_ = float(lr)
        if self._state is not None:
            self._state[1:2].fill_(self.Lr_)

    def SetGradScale(self, s: float) -> None:
        self.GradScale_ = float(s)
        if self._state is not None:
            self._state[6:7].fill_(self.GradScale_)

    def SetClipGradNorm(self, max_norm: Optional[float]) -> None:
        self._clip_norm = max_norm

    def _clip_coef(self):
        if self._clip_norm is None:
            return None
        for i, a in enumerate(self._arenas):
            K.sumsq(a.grad, self._clip_buf[0:1], accumulate=i > 0)
        K.clip_coef(self._clip_buf[0:1], self._clip_norm / max(self.GradScale_, 1e-30), self._clip_buf[1:2])
        return self._clip_buf[1:2]

    def Step(self) -> None:
        self._build()
        ctx = RT.OaContext.GetDefault()
        ctx.Add("AdamwGraphAdvance")
        K.optim_advance(self._state)
        coef = self._clip_coef()
        for a, m, v in zip(self._arenas, self._m, self._v):
            ctx.Add("AdamwGraph" if self.Decoupled else "Adam")
            K.adam_step(a.flat, a.grad, a.master, m, v, self._state, decoupled=self.Decoupled, inv_clip=coef)
        self.Step_ += 1

    def SaveTo(self, oam: OamModel) -> OaStatus:
        self._build()
        RT.OaContext.GetDefault().Sync()
        st = OamOptimizerState()
        st.Type = self.TypeName
        st.Lr, st.Beta1, st.Beta2, st.Eps, st.WeightDecay, st.Step = self.Lr_, self.Beta1_, self.Beta2_, self.Eps_, self.WeightDecay_, self.Step_
        st.AdamM = np.concatenate([a.gather(m) for a, m in zip(self._arenas, self._m)]) if self._arenas else np.zeros(0, np.float32)
        st.AdamV = np.concatenate([a.gather(v) for a, v in zip(self._arenas, self._v)]) if self._arenas else np.zeros(0, np.float32)
        oam.SetOptimizer(st)
        return OaStatus.Ok()

    def ValidateLoad(self, oam: OamModel) -> OaStatus:
        return self._validate_counts(oam, (self.TypeName,), True)

    def LoadFrom(self, oam: OamModel) -> OaStatus:
        st = self.ValidateLoad(oam)
        if not st:
            return st
        s = oam.GetOptimizer()
        self.Lr_, self.Beta1_, self.Beta2_, self.Eps_, self.WeightDecay_, self.Step_ = s.Lr, s.Beta1, s.Beta2, s.Eps, s.WeightDecay, s.Step
        pos_m = pos_v = 0
        for a, m, v in zip(self._arenas, self._m, self._v):
            pos_m = a.scatter(m, s.AdamM, pos_m)
            pos_v = a.scatter(v, s.AdamV, pos_v)
            a.reseed_master()
        self._state.copy_(torch.tensor([float(self.Step_), self.Lr_, self.Beta1_, self.Beta2_, self.Eps_, self.WeightDecay_,
                                        self.GradScale_, 0.0], dtype=torch.float32))
        return OaStatus.Ok()


class OaAdam(_AdamBase):
    TypeName = "Adam"
    Decoupled = False

    def __init__(self, params, lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8):
        super().__init__(params, lr, beta1, beta2, eps, 0.0)


class OaAdamW(_AdamBase):
    TypeName = "AdamW"
    Decoupled = True

    def __init__(self, params, lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.01):
        super().__init__(params, lr, beta1, beta2, eps, weight_decay)


class OaSGD(OaOptimizer):
    TypeName = "SGD"

    def __init__(self, params, lr=1e-2, momentum=0.0, weight_decay=0.0):
        super().__init__(params, lr)
        self.Momentum_, self.WeightDecay_ = float(momentum), float(weight_decay)
        self._mom: list = []

    def _init_state(self) -> None:
        self._mom = [torch.zeros(a.numel, dtype=torch.float32, device=a.device) if self.Momentum_ != 0.0 else None
                     for a in self._arenas]
        for a in self._arenas:
            a.ensure_master()

    def Step(self) -> None:
        self._build()
        RT.OaContext.GetDefault().MarkReplayUnsafe("OaSGD.Step passes the learning rate, momentum and weight decay as launch "
                                                   "arguments: a replay would ignore SetLr")
        for a, mom in zip(self._arenas, self._mom):
            RT.OaContext.GetDefault().Add("SgdMomentum" if mom is not None else "Sgd")
            K.sgd_step(a.flat, a.grad, a.master, mom, lr=self.Lr_, momentum=self.Momentum_, weight_decay=self.WeightDecay_)
        self.Step_ += 1

    def SaveTo(self, oam: OamModel) -> OaStatus:
        self._build()
        RT.OaContext.GetDefault().Sync()
        st = OamOptimizerState()
        st.Type, st.Lr, st.Beta1, st.WeightDecay, st.Step = "SGD", self.Lr_, self.Momentum_, self.WeightDecay_, self.Step_
        if self.Momentum_ != 0.0:
            st.AdamM = np.concatenate([a.gather(m) for a, m in zip(self._arenas, self._mom)])
        oam.SetOptimizer(st)
        return OaStatus.Ok()

    def ValidateLoad(self, oam: OamModel) -> OaStatus:
        if not oam.HasOptimizer() or oam.GetOptimizer().Type != "SGD":
            return OaStatus.Error(OaStatusCode.InvalidArgument, "checkpoint optimizer is not SGD")
        n = oam.GetOptimizer().AdamM.size
        if n not in (0, self._num_unpadded()):
            return OaStatus.Error(OaStatusCode.InvalidArgument, "SGD momentum size mismatch")
        return OaStatus.Ok()

    def LoadFrom(self, oam: OamModel) -> OaStatus:
        st = self.ValidateLoad(oam)
        if not st:
            return st
        s = oam.GetOptimizer()
        self.Lr_, self.Step_ = s.Lr, s.Step
        pos = 0
        for a, mom in zip(self._arenas, self._mom):
            if mom is not None and s.AdamM.size:
                pos = a.scatter(mom, s.AdamM, pos)
            a.reseed_master()
        return OaStatus.Ok()


_NS_A, _NS_B, _NS_C = 3.4445, -4.7750, 2.0315


def MoonshotScale(rows: int, cols: int, rms_match: float = 0.2) -> float:
    return rms_match * math.sqrt(max(rows, cols))


def NewtonSchulz5(update: torch.Tensor, steps: int = 5, eps: float = 1e-7) -> torch.Tensor:
    """Orthogonalises a [rows, cols] fp32 matrix with the quintic Newton-Schulz iteration
    (Source/Private/Oa/Ml/Optim/MuonRef.cpp:95-170): Z <- aZ + (bA + cA^2)Z with A = Z Z^T."""
    rows, cols = update.shape
    transposed = rows > cols
    z = K.contiguous(update.t()) if transposed else update
    ss = torch.zeros(1, dtype=torch.float32, device=z.device)
    K.sumsq(z, ss)
    z = z / torch.sqrt(ss + eps)
    for _ in range(steps):
        a = K.gemm(z, z)                       # Z Z^T           [r, r]
        aa = K.gemm(a, a, b_mn=True)           # A A             [r, r]
        b = K.binary("add", K.unary("scale", a, _NS_B), K.unary("scale", aa, _NS_C))
        z = K.binary("add", K.unary("scale", z, _NS_A), K.gemm(b, z, b_mn=True))
    return K.contiguous(z.t()) if transposed else z


class OaMuon(OaOptimizer):
    """Muon: Nesterov momentum + Newton-Schulz-5 for 2-D parameters, momentum SGD with decoupled decay for the rest."""
    TypeName = "Muon"

    def __init__(self, params, lr=1e-3, beta=0.95, weight_decay=0.1, eps=1e-8, ns5_iterations=5):
        super().__init__(params, lr)
        self.Beta_, self.WeightDecay_, self.Eps_, self.NS5Iterations_ = float(beta), float(weight_decay), float(eps), int(ns5_iterations)
        self._mom: list = []

    def _init_state(self) -> None:
        self._mom = [torch.zeros(a.numel, dtype=torch.float32, device=a.device) for a in self._arenas]
        for a in self._arenas:
            a.ensure_master()

    def Step(self) -> None:
        self._build()
        ctx = RT.OaContext.GetDefault()
        ctx.MarkReplayUnsafe("OaMuon.Step applies host-side learning rate and momentum scalars: a replay would ignore SetLr")
        for a, mom in zip(self._arenas, self._mom):
            w_all = a.master if a.master is not None else a.flat
            for p, o in zip(a.params, a.offsets):
                n = p.NumElements()
                g = a.grad[o:o + n].float()
                m = mom[o:o + n]
                ctx.Add("MuonNesterov")
                m.mul_(self.Beta_).add_(g, alpha=1 - self.Beta_)
                nest = g * (1 - self.Beta_) + m * self.Beta_
                w = w_all[o:o + n]
                if p.Data.Rank() == 2:
                    rows, cols = p.Tensor().shape
                    ctx.Add("MuonNormalize")
                    ortho = NewtonSchulz5(nest.view(rows, cols), self.NS5Iterations_, 1e-7).reshape(-1)
                    ctx.Add("MuonApply")
                    w.mul_(1 - self.Lr_ * self.WeightDecay_).add_(ortho, alpha=-self.Lr_ * MoonshotScale(rows, cols))
                else:
                    ctx.Add("MuonVector")
                    w.mul_(1 - self.Lr_ * self.WeightDecay_).add_(nest, alpha=-self.Lr_)
            if a.master is not None:
                K.cast(a.master, a.dtype, out=a.flat)
        self.Step_ += 1

    def SaveTo(self, oam: OamModel) -> OaStatus:
        self._build()
        st = OamOptimizerState()
        st.Type, st.Lr, st.Beta1, st.WeightDecay, st.Eps, st.Step = "Muon", self.Lr_, self.Beta_, self.WeightDecay_, self.Eps_, self.Step_
        st.MuonM = np.concatenate([a.gather(m) for a, m in zip(self._arenas, self._mom)])
        st.AdamM = st.MuonM  # the count field of a Muon-only file describes the momentum vector
        oam.SetOptimizer(_muon_only(st))
        return OaStatus.Ok()

    def ValidateLoad(self, oam: OamModel) -> OaStatus:
        if not oam.HasOptimizer() or oam.GetOptimizer().Type != "Muon":
            return OaStatus.Error(OaStatusCode.InvalidArgument, "checkpoint optimizer is not Muon")
        if oam.GetOptimizer().MuonM.size != self._num_unpadded():
            return OaStatus.Error(OaStatusCode.InvalidArgument, "Muon momentum size mismatch")
        return OaStatus.Ok()

    def LoadFrom(self, oam: OamModel) -> OaStatus:
        st = self.ValidateLoad(oam)
        if not st:
            return st
        s = oam.GetOptimizer()
        self.Lr_, self.Step_ = s.Lr, s.Step
        pos = 0
        for a, mom in zip(self._arenas, self._mom):
            pos = a.scatter(mom, s.MuonM, pos)
            a.reseed_master()
        return OaStatus.Ok()


def _muon_only(st: OamOptimizerState) -> OamOptimizerState:
    out = OamOptimizerState()
    out.__dict__.update(st.__dict__)
    out.AdamM = st.MuonM
    out.AdamV = np.zeros(0, np.float32)
    out.MuonM = np.zeros(0, np.float32)
    return out


def IsMuonMatrixParam(path: str, param: OaParameter) -> bool:
    """2-D hidden matrices go to Muon; embeddings, heads, biases and 1-D parameters go to AdamW
    (Source/Private/Oa/Ml/Optim/MuonRef.cpp, IsMuonMatrixParam)."""
    if not param.RequiresGrad or param.Data.Rank() != 2:
        return False
    aux = {"embed", "wte", "token_embed", "byte_embed", "head", "lm_head", "output", "classifier", "bias"}
    return not any(seg in aux for seg in path.split("."))


class OaMuonAdamWConfig:
    def __init__(self, muon_lr=2e-2, adamw_lr=3e-4, beta=0.95, weight_decay=0.1):
        self.MuonLr, self.AdamWLr, self.Beta, self.WeightDecay = muon_lr, adamw_lr, beta, weight_decay


class OaOptimizerComposite(OaOptimizer):
    """Runs several optimizers as one (Muon for matrices + AdamW for the rest)."""
    TypeName = "MuonAdamW"

    def __init__(self):
        super().__init__([], 0.0)
        self.Children_: list[OaOptimizer] = []
        self.BaseMuonLr_, self.BaseAdamWLr_ = 2e-2, 3e-4

    @staticmethod
    def FromNamed(named, cfg: Optional[OaMuonAdamWConfig] = None) -> "OaOptimizerComposite":
        cfg = cfg or OaMuonAdamWConfig()
        muon = [n.Param for n in named if IsMuonMatrixParam(n.Name, n.Param)]
        rest = [n.Param for n in named if not IsMuonMatrixParam(n.Name, n.Param)]
        c = OaOptimizerComposite()
        c.Add(OaMuon(muon, cfg.MuonLr, cfg.Beta, cfg.WeightDecay))
        c.Add(OaAdamW(rest, cfg.AdamWLr, weight_decay=cfg.WeightDecay))
        c.InitDualLr(cfg.MuonLr, cfg.AdamWLr)
        return c

    def Add(self, opt: OaOptimizer) -> None:
        self.Children_.append(opt)

    def InitDualLr(self, muon_lr: float, adamw_lr: float) -> None:
        self.BaseMuonLr_, self.BaseAdamWLr_ = muon_lr, adamw_lr
        self.Lr_ = adamw_lr

    def SetLr(self, lr: float) -> None:
        """Scales both children by lr / base AdamW lr, keeping their ratio."""
        ratio = lr / self.BaseAdamWLr_ if self.BaseAdamWLr_ else 1.0
        self.Lr_ = lr
        for c in self.Children_:
            c.SetLr((self.BaseMuonLr_ if isinstance(c, OaMuon) else self.BaseAdamWLr_) * ratio)

    def Step(self) -> None:
        for c in self.Children_:
            c.Step()
        self.Step_ += 1

    def NotifyProgramReplay(self, count: int = 1) -> None:
        self.Step_ += count
        for c in self.Children_:
            c.NotifyProgramReplay(count)

    def ZeroGrad(self) -> None:
        for c in self.Children_:
            c.ZeroGrad()

    def SaveTo(self, oam: OamModel) -> OaStatus:
        st = OamOptimizerState()
        st.Type, st.Step, st.Lr = "MuonAdamW", self.Step_, self.Lr_
        for c in self.Children_:
            tmp = OamModel()
            c.SaveTo(tmp)
            s = tmp.GetOptimizer()
            if isinstance(c, OaMuon):
                st.MuonM = s.AdamM
                st.Beta1 = c.Beta_
            else:
                st.AdamM, st.AdamV, st.Beta2, st.Eps, st.WeightDecay = s.AdamM, s.AdamV, s.Beta2, s.Eps, s.WeightDecay
        oam.SetOptimizer(st)
        return OaStatus.Ok()

    def ValidateLoad(self, oam: OamModel) -> OaStatus:
        if not oam.HasOptimizer() or oam.GetOptimizer().Type != "MuonAdamW":
            return OaStatus.Error(OaStatusCode.InvalidArgument, "checkpoint optimizer is not MuonAdamW")
        s = oam.GetOptimizer()
        for c in self.Children_:
            n = c._num_unpadded()
            have = s.MuonM.size if isinstance(c, OaMuon) else s.AdamM.size
            if n != have:
                return OaStatus.Error(OaStatusCode.InvalidArgument, "MuonAdamW state size mismatch")
        return OaStatus.Ok()

    def LoadFrom(self, oam: OamModel) -> OaStatus:
        st = self.ValidateLoad(oam)
        if not st:
            return st
        s = oam.GetOptimizer()
        self.Step_ = s.Step
        for c in self.Children_:
            tmp = OamModel()
            sub = OamOptimizerState()
            sub.__dict__.update(s.__dict__)
            if isinstance(c, OaMuon):
                sub.Type, sub.AdamM, sub.AdamV, sub.MuonM = "Muon", s.MuonM, np.zeros(0, np.float32), np.zeros(0, np.float32)
                sub.Lr = c.Lr_
                tmp.SetOptimizer(sub)
                # a Muon-only file is read back with the momentum in MuonM
                c.Step_ = s.Step
                pos = 0
                for a, mom in zip(c.Arenas(), c._mom):
                    pos = a.scatter(mom, s.MuonM, pos)
                    a.reseed_master()
            else:
                sub.Type, sub.MuonM = c.TypeName, np.zeros(0, np.float32)
                sub.Lr = c.Lr_
                tmp.SetOptimizer(sub)
                r = c.LoadFrom(tmp)
                if not r:
                    return r
        return OaStatus.Ok()
