"""OaMamba3Module: the Mamba-3 SISO mixer (Source/Private/Oa/Ml/Nn/Mamba3/Mamba3.cpp:28-135 constructor, :160-250 Forward,
Step / ResetState below it).

Parameters, in registration order: in_proj [d_in_proj, d_model] (row blocks z | x | B | C | dd_dt | dd_A | trap | angle),
dt_bias [1, H], B_bias [H, N] (ones), C_bias [H, N] (ones), D [H] (zeros), out_proj [d_model, d_inner] and, with the
gated output norm, norm_weight [H, P].  Forward is in_proj GEMM -> one fused core op (preprocess + selective scan [+
gated per-head RMSNorm], csrc/kernels/mamba3.cu) -> out_proj GEMM; the core writes every gradient of the projected row
into one [B*S, d_in_proj] buffer, so the in_proj backward is two GEMMs on it.  Step keeps the recurrent state
(StepSsm / StepAngle / StepK / StepV in the reference) for token-by-token decoding.
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from ...core import fn_matrix as F
from ...core.matrix import OaMatrix
from ...ops import kernels as K
from ...ops import mamba3 as M3
from .. import autograd as AG
from ..module import OaModule


def _param_grad(p: OaMatrix, g32: Optional[torch.Tensor]):
    """Hands an fp32 parameter gradient to the tape in the parameter's shape and dtype."""
    if g32 is None or p is None or not p.RequiresGrad():
        return None
    t = p.Tensor()
    g = g32.reshape(t.shape)
    return g if g.dtype == t.dtype else K.cast(g.contiguous(), t.dtype)


def Mamba3Core(proj: OaMatrix, dt_bias: OaMatrix, b_bias: OaMatrix, c_bias: OaMatrix, d_skip: Optional[OaMatrix],
               norm_weight: Optional[OaMatrix], dims: M3.Mamba3Dims, batch: int, seq: int) -> OaMatrix:
    """proj [B*S, d_in_proj] -> mixed [B*S, d_inner]: preprocess, scan and (with norm_weight) the gated output norm."""
    F._ctx_add("Mamba3Siso")
    tp = F._c(proj.Tensor())
    params = [dt_bias, b_bias, c_bias, d_skip]
    pt = [m.Tensor() if m is not None else None for m in params]
    need = AG.IsEnabled() and (proj.RequiresGrad() or any(m is not None and m.RequiresGrad() for m in params + [norm_weight]))
    y, saved = M3.core_fwd(tp, pt[0], pt[1], pt[2], pt[3], dims, batch, seq, save=need)
    rstd = None
    out_t = y
    if norm_weight is not None:
        F._ctx_add("Mamba3GatedNorm")
        out_t, rstd = M3.gated_norm_fwd(y, tp, norm_weight.Tensor(), dims)
    out = OaMatrix(out_t)

    def back(g):
        F._ctx_add("Mamba3SisoBwd")
        g = F._c(g)
        dproj = torch.empty_like(tp)
        dnw = None
        if norm_weight is not None:
            g, dnw = M3.gated_norm_bwd(y, tp, norm_weight.Tensor(), rstd, g, dims, dproj)
        dproj, ddtb, dBb, dCb, dD = M3.core_bwd(saved, g, dproj)
        return (dproj, _param_grad(dt_bias, ddtb), _param_grad(b_bias, dBb), _param_grad(c_bias, dCb), _param_grad(d_skip, dD),
                _param_grad(norm_weight, dnw))

    return AG.attach("Mamba3Siso", out, [proj, dt_bias, b_bias, c_bias, d_skip, norm_weight], back)


class OaMamba3Module(OaModule):
    def __init__(self, d_model: int, d_state: int = 128, expand: int = 2, headdim: int = 64, ngroups: int = 1,
                 rope_fraction: float = 0.5, is_mimo: bool = False, mimo_rank: int = 4, dt_min: float = 1e-3, dt_max: float = 0.1,
                 dt_init_floor: float = 1e-4, a_floor: float = 1e-4, is_outproj_norm: bool = False, chunk: int = 256):
        super().__init__()
        if is_mimo:
            raise NotImplementedError("the MIMO variant of Mamba-3 is not built; use is_mimo=False")
        if ngroups != 1:
            raise NotImplementedError("Mamba-3 with ngroups != 1 is not built")
        self.DModel, self.DState, self.Expand, self.HeadDim = d_model, d_state, expand, headdim
        self.DInner = expand * d_model
        if self.DInner % headdim:
            raise ValueError("expand * d_model must be a multiple of headdim")
        self.NHeads = self.DInner // headdim
        self.RopeDim = int(d_state * rope_fraction) & ~1
        self.NumRopeAngles = self.RopeDim // 2
        self.IsOutprojNorm = is_outproj_norm
        self.Dims = M3.Mamba3Dims(self.DInner, self.NHeads, headdim, d_state, self.NumRopeAngles, has_z=not is_outproj_norm,
                                  dt_min=dt_min, dt_max=dt_max, afloor=a_floor, chunk=chunk)
        H = self.NHeads
        self.InProj = self.RegisterParameter("in_proj", F.RandGlorotUniform([self.Dims.d_in_proj, d_model]))
        # dt_bias = inverse softplus of dt drawn log-uniformly from [dt_min, dt_max] and floored
        r = F.Rand([H], torch.float32).Tensor().float().cpu()
        dtv = torch.exp(r * (math.log(dt_max) - math.log(dt_min)) + math.log(dt_min)).clamp_min(dt_init_floor)
        dt_bias = dtv + torch.log(-torch.expm1(-dtv))
        wdev = self.InProj.Data.Tensor().device
        self.DtBias = self.RegisterParameter("dt_bias", OaMatrix(dt_bias.reshape(1, H).to(wdev)))
        self.BBias = self.RegisterParameter("B_bias", F.Ones([H, d_state], torch.float32))
        self.CBias = self.RegisterParameter("C_bias", F.Ones([H, d_state], torch.float32))
        self.D = self.RegisterParameter("D", F.Zeros([H], torch.float32))
        self.OutProj = self.RegisterParameter("out_proj", F.RandGlorotUniform([d_model, self.DInner]))
        self.NormWeight = self.RegisterParameter("norm_weight", F.Ones([H, headdim], torch.float32)) if is_outproj_norm else None
        self._state: Optional[dict] = None

    # ---- training / prefill
    def Forward(self, x: OaMatrix) -> OaMatrix:
        if x.Rank() != 3:
            raise ValueError(f"OaMamba3Module.Forward expects rank-3 [batch, seq, d_model], got rank {x.Rank()}")
        batch, seq = x.Size(0), x.Size(1)
        flat = x.Reshape([batch * seq, self.DModel])
        proj = F.Linear(flat, self.InProj.Data, None, name="Mamba3InProj")
        mixed = Mamba3Core(proj, self.DtBias.Data, self.BBias.Data, self.CBias.Data, self.D.Data,
                           self.NormWeight.Data if self.NormWeight is not None else None, self.Dims, batch, seq)
        out = F.Linear(mixed, self.OutProj.Data, None, name="Mamba3OutProj")
        return out.Reshape([batch, seq, self.DModel])

    # ---- decoding
    def ResetState(self, batch: int = 0) -> None:
        """Drops the recurrent decode state; the next Step allocates it for whatever batch it receives."""
        self._state = None

    def Step(self, x: OaMatrix) -> OaMatrix:
        """x [batch, d_model] -> [batch, d_model]; the recurrent state lives in the module until ResetState()."""
        if self._state is None:
            self._state = {}
        with AG.OaGradNo():
            proj = F.Linear(x, self.InProj.Data, None, name="Mamba3InProj")
            tp = F._c(proj.Tensor())
            y = M3.step(tp, self.DtBias.Data.Tensor(), self.BBias.Data.Tensor(), self.CBias.Data.Tensor(), self.D.Data.Tensor(),
                        self.Dims, self._state)
            if self.NormWeight is not None:
                y, _ = M3.gated_norm_fwd(y, tp, self.NormWeight.Data.Tensor(), self.Dims)
            return F.Linear(OaMatrix(y), self.OutProj.Data, None, name="Mamba3OutProj")

    def Prefill(self, x: OaMatrix) -> OaMatrix:
        """Forward over a prompt [batch, seq, d_model] that also leaves the decode state behind (no autograd)."""
        batch, seq = x.Size(0), x.Size(1)
        self._state = {}
        with AG.OaGradNo():
            proj = F.Linear(x.Reshape([batch * seq, self.DModel]), self.InProj.Data, None, name="Mamba3InProj")
            tp = F._c(proj.Tensor())
            y, _ = M3.core_fwd(tp, self.DtBias.Data.Tensor(), self.BBias.Data.Tensor(), self.CBias.Data.Tensor(), self.D.Data.Tensor(),
                               self.Dims, batch, seq, save=False, final=self._state)
            if self.NormWeight is not None:
                y, _ = M3.gated_norm_fwd(y, tp, self.NormWeight.Data.Tensor(), self.Dims)
            out = F.Linear(OaMatrix(y), self.OutProj.Data, None, name="Mamba3OutProj")
        return out.Reshape([batch, seq, self.DModel])
