"""Mamba-3 language model: embedding -> N x (RMSNorm -> OaMamba3Module -> + residual) -> RMSNorm -> head.

The mixer is the reference's OaMamba3Module (Source/Private/Oa/Ml/Nn/Mamba3/Mamba3.cpp); the reference's own LM around
it is the one-block model of the NLP suite (Source/Private/Oa/Ml/NlpSuite.cpp, Mamba3 arch), stacked here.
Checkpoint names: `embed.weight`, `blocks.<i>.norm.weight`, `blocks.<i>.mixer.<in_proj|dt_bias|B_bias|C_bias|D|out_proj
[|norm_weight]>`, `ln_final.weight`, `head.weight`.
"""
from __future__ import annotations

import struct
from dataclasses import dataclass
from typing import Optional

from ..core import fn_matrix as F
from ..core.matrix import OaMatrix
from ..ml import fn_loss as L
from ..ml.module import OaModule
from ..ml.nn.layers import OaEmbedding, OaLinear, OaRmsNorm
from ..ml.nn.mamba3 import OaMamba3Module


@dataclass
class OaMamba3Config:
    Vocab: int = 32000
    DModel: int = 1536
    NLayers: int = 32
    DState: int = 128
    Expand: int = 2
    HeadDim: int = 64
    SeqLen: int = 4096
    Chunk: int = 256
    OutprojNorm: bool = True
    Eps: float = 1e-5
    InitStd: Optional[float] = 0.02
    ConvWidth: int = 0            # > 0: causal depthwise convolution + SiLU over x | B | C before the scan
    ALog: bool = False            # learned per-head decay A = -exp(A_log), A_log ~ log U(1, 16), instead of the data-dependent one

    @staticmethod
    def Mamba3_32x1536() -> "OaMamba3Config":
        """vocab 32000, d 1536, 32 layers, state 128, expand 2, head dim 64, conv width 4, A_log ~ log U(1, 16),
        dt log-uniform in [1e-3, 1e-1], seq 4096."""
        return OaMamba3Config(ConvWidth=4, ALog=True)

    @staticmethod
    def Tiny() -> "OaMamba3Config":
        return OaMamba3Config(256, 32, 2, 32, 2, 16, 64, 16)


class OaMamba3Block(OaModule):
    def __init__(self, cfg: OaMamba3Config):
        super().__init__()
        self.Norm = self.RegisterModule("norm", OaRmsNorm(cfg.DModel, cfg.Eps))
        self.Mixer = self.RegisterModule("mixer", OaMamba3Module(cfg.DModel, cfg.DState, cfg.Expand, cfg.HeadDim,
                                                                 is_outproj_norm=cfg.OutprojNorm, chunk=cfg.Chunk,
                                                                 conv_width=cfg.ConvWidth, a_log=cfg.ALog))

    def Forward(self, x: OaMatrix) -> OaMatrix:
        return F.Add(x, self.Mixer.Forward(self.Norm.Forward(x)))

    def Step(self, x: OaMatrix) -> OaMatrix:
        return F.Add(x, self.Mixer.Step(self.Norm.Forward(x)))


class OaMamba3LmModel(OaModule):
    def __init__(self, cfg: OaMamba3Config):
        super().__init__()
        self.Cfg = cfg
        self.Embed = self.RegisterModule("embed", OaEmbedding(cfg.Vocab, cfg.DModel, cfg.InitStd))
        self.Blocks = []
        blocks = OaModule()
        for i in range(cfg.NLayers):
            b = OaMamba3Block(cfg)
            blocks.RegisterModule(str(i), b)
            self.Blocks.append(b)
        self.RegisterModule("blocks", blocks)
        self.LnFinal = self.RegisterModule("ln_final", OaRmsNorm(cfg.DModel, cfg.Eps))
        self.Head = self.RegisterModule("head", OaLinear(cfg.DModel, cfg.Vocab, False, cfg.InitStd))

    def Forward(self, ids: OaMatrix) -> OaMatrix:
        """ids [B, S] int32 -> logits [B*S, vocab]."""
        batch, seq = ids.Size(0), ids.Size(1)
        x = F.Embedding(self.Embed.Weight.Data, ids, None, seq).Reshape([batch, seq, self.Cfg.DModel])
        for b in self.Blocks:
            x = b.Forward(x)
        x = self.LnFinal.Forward(x.Reshape([batch * seq, self.Cfg.DModel]))
        return self.Head.Forward(x)

    def Loss(self, ids: OaMatrix, targets: OaMatrix) -> OaMatrix:
        logits = self.Forward(ids)
        return L.CrossEntropy(logits, targets.Reshape([targets.NumElements()]), in_place_grad=True)

    def ResetState(self) -> None:
        for b in self.Blocks:
            b.Mixer.ResetState()

    def Step(self, ids: OaMatrix) -> OaMatrix:
        """ids [B, 1] -> logits [B, vocab] using the recurrent state of every block (constant cost per token)."""
        batch = ids.Size(0)
        x = F.Embedding(self.Embed.Weight.Data, ids, None, 1).Reshape([batch, self.Cfg.DModel])
        for b in self.Blocks:
            x = b.Step(x)
        return self.Head.Forward(self.LnFinal.Forward(x))

    def OamConfig(self) -> dict:
        c = self.Cfg
        blob = struct.pack("<8I", c.Vocab, c.DModel, c.NLayers, c.DState, c.Expand, c.HeadDim, c.SeqLen, int(c.OutprojNorm))
        return {"Architecture": "OaMamba3Lm", "DModel": c.DModel, "NLayers": c.NLayers, "DVocab": c.Vocab, "ArchConfig": blob}

    def FlopsPerToken(self) -> float:
        """Training FLOPs per token: projections and head as GEMMs (x3 for forward + backward), scan as 6*P*N per head-row."""
        c = self.Cfg
        d_inner = c.Expand * c.DModel
        heads = d_inner // c.HeadDim
        d_in_proj = 2 * d_inner + 2 * c.DState + 3 * heads + (int(c.DState * 0.5) & ~1) // 2
        per_layer = 2 * c.DModel * (d_in_proj + d_inner) + 6 * d_inner * c.DState
        return 3.0 * (c.NLayers * per_layer + 2 * c.DModel * c.Vocab)
