"""OaEmpyrealmCore / OaEmpyrealmModule: the Empyrealm sequence-modelling backbone.

Reference: Source/Public/Oa/Ml/Nn/Empyrealm/EmpyrealmCore.h:33-117 and Source/Private/Oa/Ml/Nn/Empyrealm/
EmpyrealmCore.cpp, EmpyrealmModule.{h,cpp}.  In the reference the Empyrealm kernels (EmpyrealmDt / EmpyrealmAdt /
EmpyrealmSiso) are renamed copies of the Mamba-3 kernels with identical code, kept apart so the architecture can diverge
later; here the mixer is the same selective-scan implementation under its own class name, so checkpoints carry the
`mixer.*` parameter names of the reference.  The core is: input projection (byte / token embedding, a caller-supplied
module, or none) -> mixer -> per-token residual -> flat [B*S, DModel] features.
"""
from __future__ import annotations

from typing import Optional

from ...core import fn_matrix as F
from ...core.matrix import OaMatrix
from ..module import OaModule
from .layers import OaEmbedding
from .mamba3 import OaMamba3Module


class OaEmpyrealmModule(OaMamba3Module):
    """The Empyrealm mixer: selective state-space scan with trapezoidal update, rotary state and gated output."""


class OaEmpyrealmCore(OaModule):
    def __init__(self, embed=None, d_model: int = 0, d_state: int = 32, expand: int = 2, headdim: int = 16, ngroups: int = 1,
                 rope_fraction: float = 0.5, is_mimo: bool = False, mimo_rank: int = 1, dt_min: float = 1e-3, dt_max: float = 0.1,
                 dt_init_floor: float = 1e-4, a_floor: float = 1e-4, is_outproj_norm: bool = True):
        """`embed` selects the input mode: an int is a vocabulary size (Forward takes [B, S] token / byte indices and the
        core owns an OaEmbedding child `embed`), an OaModule is a custom projection that must return [B, S, DModel]
        (or flat [B*S, DModel]), None is the embedded-only mode (no embed parameters exist; use ForwardEmbedded)."""
        super().__init__()
        if d_model <= 0:
            raise ValueError("OaEmpyrealmCore needs a positive model width")
        self.DModel = d_model
        self.IsByteMode = isinstance(embed, int)
        self.Embed = None
        if self.IsByteMode:
            self.Embed = self.RegisterModule("embed", OaEmbedding(int(embed), d_model))
        elif embed is not None:
            self.Embed = self.RegisterModule("embed", embed)
        self.Mixer_ = self.RegisterModule("mixer", OaEmpyrealmModule(d_model, d_state, expand, headdim, ngroups, rope_fraction, is_mimo,
                                                                     mimo_rank, dt_min, dt_max, dt_init_floor, a_floor, is_outproj_norm))

    @staticmethod
    def EmbeddedOnly(d_model: int, **kw) -> "OaEmpyrealmCore":
        return OaEmpyrealmCore(None, d_model, **kw)

    def Forward(self, x: OaMatrix) -> OaMatrix:
        if self.Embed is None:
            raise RuntimeError("OaEmpyrealmCore.Forward called in embedded-only mode; use ForwardEmbedded with [B, S, D] features")
        emb = self.Embed.Forward(x)
        if x.Rank() == 2 and emb.Rank() == 2 and self.IsByteMode:
            emb = F.Reshape(emb, [x.Size(0), x.Size(1), self.DModel])   # B independent length-S scans, not one of length B*S
        return self.ForwardEmbedded(emb)

    def ForwardEmbedded(self, embedded: OaMatrix) -> OaMatrix:
        """Mixer + residual on [B, S, D] (or flat [B*S, D], taken as one sequence); returns flat [B*S, D]."""
        if embedded.Rank() == 3:
            batch, seq = embedded.Size(0), embedded.Size(1)
            e3 = embedded
        else:
            batch, seq = 1, embedded.Size(0)
            e3 = F.Reshape(embedded, [1, seq, self.DModel])
        flat = F.Reshape(e3, [batch * seq, self.DModel])
        mixed = F.Reshape(self.Mixer_.Forward(e3), [batch * seq, self.DModel])
        return F.Add(mixed, flat)

    def Mixer(self) -> OaEmpyrealmModule:
        return self.Mixer_

    def ResetState(self, batch: int) -> None:
        self.Mixer_.ResetState(batch)
