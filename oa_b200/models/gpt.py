"""Decoder-only Transformer language models built from OaTransformerBlock.

Covers the char-level pre-LayerNorm model with learned positions (the shape of the reference's canonical
Transformer LM, Source/Private/Oa/Ml/NlpSuite.cpp:165-224, stacked N times), the GPT-style RMSNorm + RoPE
model and the 7B-class SwiGLU model.  Checkpoint names: `embed.weight`, `pos_embed.weight`,
`blocks.<i>.<...>`, `ln_final.weight[/bias]`, `head.weight[/bias]`.
"""
from __future__ import annotations

import struct
from dataclasses import dataclass
from typing import Optional

from ..core import fn_matrix as F
from ..core.matrix import OaMatrix
from ..ml import fn_loss as L
from ..ml.module import OaModule
from ..ml.nn.layers import OaEmbedding, OaLayerNorm, OaLinear, OaRmsNorm, OaTransformerBlock
from ..ml.nn.moe import OaMoE


@dataclass
class OaGptConfig:
    Vocab: int = 256
    DModel: int = 128
    NLayers: int = 4
    NHeads: int = 4
    DFf: int = 512
    SeqLen: int = 128
    Norm: str = "layer"          # "layer" | "rms"
    Ffn: str = "gelu"            # "gelu" | "swiglu"
    RopeTheta: float = 0.0       # 0: learned positions
    Bias: bool = True
    Eps: float = 1e-5
    InitStd: Optional[float] = 0.02
    NumExperts: int = 0          # > 0: every block's FFN is a sparse MoE layer
    TopK: int = 2
    ExpertFf: int = 0
    SharedExperts: int = 0
    AuxAlpha: float = 0.0
    ExpertBias: bool = True

    @staticmethod
    def CharLm() -> "OaGptConfig":
        """vocab 256, d 128, 4 layers, 4 heads, FFN 512 GELU, pre-LayerNorm, learned positions, seq 128."""
        return OaGptConfig()

    @staticmethod
    def Gpt350M() -> "OaGptConfig":
        """vocab 32000, d 1024, 24 layers, 16 heads (head_dim 64), FFN 4096 GELU, RMSNorm, RoPE, seq 2048."""
        return OaGptConfig(32000, 1024, 24, 16, 4096, 2048, "rms", "gelu", 10000.0, False, 1e-5, 0.02)

    @staticmethod
    def Moe16x2048() -> "OaGptConfig":
        """vocab 32000, d 2048, 16 layers, 16 heads, 64 experts top-2 (softmax router), SwiGLU expert FFN 1408, one shared
        expert, load-balance loss 0.01, RMSNorm, RoPE, seq 2048."""
        return OaGptConfig(32000, 2048, 16, 16, 1408, 2048, "rms", "swiglu", 10000.0, False, 1e-5, 0.02, NumExperts=64, TopK=2,
                           ExpertFf=1408, SharedExperts=1, AuxAlpha=0.01, ExpertBias=False)

    @staticmethod
    def Llama7B() -> "OaGptConfig":
        """vocab 32000, d 4096, 32 layers, 32 heads, SwiGLU FFN 11008, RMSNorm, RoPE, seq 4096."""
        return OaGptConfig(32000, 4096, 32, 32, 11008, 4096, "rms", "swiglu", 10000.0, False, 1e-5, 0.02)


class OaGptModel(OaModule):
    def __init__(self, cfg: OaGptConfig):
        super().__init__()
        self.Cfg = cfg
        self.Embed = self.RegisterModule("embed", OaEmbedding(cfg.Vocab, cfg.DModel, cfg.InitStd))
        self.PosEmbed = None
        if cfg.RopeTheta <= 0:
            self.PosEmbed = self.RegisterModule("pos_embed", OaEmbedding(cfg.SeqLen, cfg.DModel, cfg.InitStd))
        self.Blocks = []
        blocks = OaModule()
        for i in range(cfg.NLayers):
            moe = None
            if cfg.NumExperts > 0:
                moe = OaMoE(cfg.DModel, cfg.ExpertFf or cfg.DFf, cfg.NumExperts, cfg.TopK, cfg.Eps, cfg.SharedExperts, cfg.InitStd,
                            expert_bias=cfg.ExpertBias)
                moe.SetAuxLossAlpha(cfg.AuxAlpha)
            b = OaTransformerBlock(cfg.DModel, cfg.DFf, cfg.SeqLen, cfg.NHeads, cfg.Eps, norm=cfg.Norm, ffn=cfg.Ffn, bias=cfg.Bias,
                                   rope_theta=cfg.RopeTheta, init_std=cfg.InitStd, moe=moe)
            blocks.RegisterModule(str(i), b)
            self.Blocks.append(b)
        self.RegisterModule("blocks", blocks)
        self.LnFinal = self.RegisterModule("ln_final", OaLayerNorm(cfg.DModel, cfg.Eps) if cfg.Norm == "layer" else OaRmsNorm(cfg.DModel, cfg.Eps))
        self.Head = self.RegisterModule("head", OaLinear(cfg.DModel, cfg.Vocab, cfg.Bias, cfg.InitStd))

    def Hidden(self, ids: OaMatrix) -> OaMatrix:
        batch, seq = ids.Size(0), ids.Size(1)
        x = F.Embedding(self.Embed.Weight.Data, ids, self.PosEmbed.Weight.Data if self.PosEmbed else None, seq)
        for b in self.Blocks:
            x = b.Forward(x, batch, seq)
        return self.LnFinal.Forward(x)

    def Forward(self, ids: OaMatrix) -> OaMatrix:
        """ids [B, S] int32 -> logits [B*S, vocab]."""
        return self.Head.Forward(self.Hidden(ids))

    def Loss(self, ids: OaMatrix, targets: OaMatrix) -> OaMatrix:
        """Mean next-token cross-entropy; the logits buffer is reused for its own gradient."""
        logits = self.Forward(ids)
        loss = L.CrossEntropy(logits, targets.Reshape([targets.NumElements()]), in_place_grad=True)
        if self.Cfg.NumExperts > 0 and self.Cfg.AuxAlpha > 0:
            for b in self.Blocks:
                loss = F.Add(loss, b.Moe.AuxLoss())
        return loss

    def OamConfig(self) -> dict:
        c = self.Cfg
        blob = struct.pack("<8I", c.Vocab, c.DModel, c.NLayers, c.NHeads, c.DFf, c.SeqLen, int(c.Norm == "rms"), int(c.Ffn == "swiglu"))
        return {"Architecture": "OaGpt", "DModel": c.DModel, "NLayers": c.NLayers, "DVocab": c.Vocab, "ArchConfig": blob}

    def FlopsPerToken(self) -> float:
        """Training FLOPs per token (forward + backward = 3x forward), attention counted causal."""
        c = self.Cfg
        ffn_mats = 3 if c.Ffn == "swiglu" else 2
        ffn = ffn_mats * c.DModel * c.DFf
        if c.NumExperts > 0:
            ffn = 3 * c.DModel * (c.ExpertFf or c.DFf) * (c.TopK + c.SharedExperts) + c.DModel * c.NumExperts
        per_layer = 2 * (4 * c.DModel * c.DModel + ffn) + 2 * 2 * c.SeqLen * c.DModel / 2
        return 3.0 * (c.NLayers * per_layer + 2 * c.DModel * c.Vocab)
