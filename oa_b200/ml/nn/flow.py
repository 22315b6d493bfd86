"""Flow-matching / diffusion backbone: sinusoidal time embedding, bidirectional adaptive-LayerNorm transformer, denoiser.

Reference: Source/Public/Oa/Ml/Nn/Flow/{FlowTimeEmbedding,FlowTransformer,FlowDenoiser}.h and
Source/Private/Oa/Ml/Nn/Flow/*.cpp.  Blocks are OaTransformerBlock in bidirectional mode with AdaLN-Zero conditioning
(Transformer.cpp:93-147); the denoiser adds input / condition / output projections, a learned position table, per-sample
condition dropout for classifier-free guidance and the guided forward uncond + scale * (cond - uncond).
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Optional

import torch

from ...core import fn_matrix as F
from ...core.matrix import OaMatrix
from ..module import OaModule
from .layers import OaAttentionMode, OaLayerNorm, OaLinear, OaTransformerBlock


class OaFlowTimeEmbedding(OaModule):
    """t [B] or [B, 1] -> [B, dim]: sin(t f) | cos(t f) with f_i = scale * max_period^(-i / half)."""

    def __init__(self, embedding_dim: int, max_period: float = 10000.0, time_scale: float = 1000.0):
        super().__init__()
        if embedding_dim <= 0 or embedding_dim % 2 or not math.isfinite(max_period) or max_period <= 1.0 \
                or not math.isfinite(time_scale) or time_scale <= 0.0:
            raise ValueError("FlowTimeEmbedding requires positive even dimension, max period > 1 and positive scale")
        self.EmbeddingDim_, self.MaxPeriod_, self.TimeScale_ = embedding_dim, max_period, time_scale
        half = embedding_dim // 2
        freq = [time_scale * math.exp(-math.log(max_period) * i / half) for i in range(half)]
        self.Frequencies_ = F.FromFloats(freq, [1, half], torch.float32)
        self.RegisterBuffer("frequencies", self.Frequencies_, False)

    def Forward(self, time: OaMatrix) -> OaMatrix:
        if time.Rank() < 1 or time.Rank() > 2 or (time.Rank() == 2 and time.Size(1) != 1):
            raise ValueError("FlowTimeEmbedding expects [B] or [B,1]")
        t = F.Reshape(time, [time.Size(0), 1])
        if t.Tensor().dtype != torch.float32:
            t = F.Cast(t, torch.float32)
        phase = F.Mul(t, self.Frequencies_)
        return F.Concat([F.Sin(phase), F.Cos(phase)], 1)

    def EmbeddingDim(self) -> int: return self.EmbeddingDim_
    def MaxPeriod(self) -> float: return self.MaxPeriod_
    def TimeScale(self) -> float: return self.TimeScale_


@dataclass
class OaFlowTransformerConfig:
    DModel: int = 0
    HiddenDim: int = 0
    SequenceLength: int = 0
    NumLayers: int = 1
    NumHeads: int = 1
    NumExperts: int = 0
    ExpertsPerToken: int = 0
    Epsilon: float = 1e-5
    AdaptiveConditioning: bool = True


class OaFlowTransformer(OaModule):
    def __init__(self, config: OaFlowTransformerConfig):
        super().__init__()
        c = config
        if min(c.DModel, c.HiddenDim, c.SequenceLength, c.NumLayers, c.NumHeads) <= 0 or c.DModel % c.NumHeads or c.Epsilon <= 0:
            raise ValueError("FlowTransformer requires positive dimensions, layers and epsilon, with DModel divisible by NumHeads")
        if c.NumExperts < 0 or c.ExpertsPerToken < 0 or (c.NumExperts == 0 and c.ExpertsPerToken != 0) \
                or (c.NumExperts > 0 and not 0 < c.ExpertsPerToken <= c.NumExperts):
            raise ValueError("FlowTransformer MoE requires 0/0 experts for dense or 0 < ExpertsPerToken <= NumExperts")
        self.Config_ = c
        self.Blocks_ = []
        for i in range(c.NumLayers):
            moe = None
            if c.NumExperts > 0:
                from .moe import OaMoE
                moe = OaMoE(c.DModel, c.HiddenDim, c.NumExperts, c.ExpertsPerToken)
            b = OaTransformerBlock(c.DModel, c.HiddenDim, c.SequenceLength, c.NumHeads, c.Epsilon, moe=moe)
            b.SetAttentionMode(OaAttentionMode.Bidirectional)
            if c.AdaptiveConditioning:
                b.EnableAdaptiveConditioning(c.DModel)
            self.Blocks_.append(self.RegisterModule(f"block{i}", b))
        self.OutputNorm_ = self.RegisterModule("output_norm", OaLayerNorm(c.DModel, c.Epsilon))

    def Forward(self, tokens: OaMatrix) -> OaMatrix:
        return self._impl(tokens, None, None)

    def ForwardMasked(self, tokens: OaMatrix, token_mask: OaMatrix) -> OaMatrix:
        return self._impl(tokens, token_mask, None)

    def ForwardConditioned(self, tokens: OaMatrix, condition: OaMatrix, token_mask: Optional[OaMatrix] = None) -> OaMatrix:
        return self._impl(tokens, token_mask, condition)

    def _impl(self, tokens: OaMatrix, token_mask: Optional[OaMatrix], condition: Optional[OaMatrix]) -> OaMatrix:
        c = self.Config_
        if tokens.Rank() not in (2, 3):
            raise ValueError("FlowTransformer expects [B*S,D] or [B,S,D] tokens")
        batched = tokens.Rank() == 3
        rows = tokens.Size(0) * tokens.Size(1) if batched else tokens.Size(0)
        seq = tokens.Size(1) if batched else c.SequenceLength
        if seq != c.SequenceLength or tokens.Size(-1) != c.DModel or rows % c.SequenceLength:
            raise ValueError("FlowTransformer token shape does not match configured sequence length and model dimension")
        batch = rows // c.SequenceLength
        if condition is not None and (not c.AdaptiveConditioning or condition.Rank() != 2 or condition.Size(0) != batch
                                      or condition.Size(1) != c.DModel or condition.Tensor().dtype != tokens.Tensor().dtype):
            raise ValueError("FlowTransformer condition must match enabled [B,DModel] adaptive conditioning")
        additive = None
        if token_mask is not None:
            shape = tuple(token_mask.Tensor().shape)
            if shape not in ((batch, seq), (batch, seq, 1)) or token_mask.Tensor().dtype != tokens.Tensor().dtype:
                raise ValueError("FlowTransformer token mask must match [B,S] or [B,S,1] and token dtype")
            key = F.Scale(F.AddScalar(F.Reshape(token_mask, [batch, 1, seq]), -1.0), 1.0e4)           # 0 keep, -1e4 drop
            additive = F.Reshape(F.RepeatInterleave(key, c.NumHeads * seq, 1), [batch * c.NumHeads * seq, seq])
        out = F.Reshape(tokens, [rows, c.DModel]) if batched else tokens
        for b in self.Blocks_:
            if condition is not None:
                out = b.ForwardConditioned(out, condition, additive)
            else:
                out = b.Forward(out, batch, seq, 0, additive)
        out = self.OutputNorm_.Forward(out)
        return F.Reshape(out, list(tokens.Tensor().shape)) if batched else out

    def SetSequenceLength(self, seq: int) -> None:
        if seq <= 0:
            raise ValueError("FlowTransformer sequence length must be positive")
        self.Config_.SequenceLength = seq
        for b in self.Blocks_:
            b.SetSeqLen(seq)

    def Config(self) -> OaFlowTransformerConfig: return self.Config_
    def IsMoe(self) -> bool: return self.Config_.NumExperts > 0
    def NumLayers(self) -> int: return self.Config_.NumLayers

    def Block(self, index: int) -> OaTransformerBlock:
        if not 0 <= index < self.Config_.NumLayers:
            raise IndexError("FlowTransformer block index is out of range")
        return self.Blocks_[index]


@dataclass
class OaFlowDenoiserConfig:
    InputDim: int = 0
    ConditionDim: int = 0
    Backbone: OaFlowTransformerConfig = field(default_factory=OaFlowTransformerConfig)
    TimeMaxPeriod: float = 10000.0
    TimeScale: float = 1000.0
    ConditionDropoutP: float = 0.0     # per-sample conditioning dropout in training (classifier-free guidance); time is never dropped


class OaFlowDenoiser(OaModule):
    """sample [B, S, InputDim] (+ time [B], condition [B, ConditionDim], token mask [B, S]) -> velocity / noise [B, S, InputDim]."""

    def __init__(self, config: OaFlowDenoiserConfig):
        super().__init__()
        c, bb = config, config.Backbone
        if c.InputDim <= 0 or c.ConditionDim < 0 or not 0.0 <= c.ConditionDropoutP < 1.0:
            raise ValueError("FlowDenoiser requires a positive input dimension, non-negative condition dimension and dropout in [0,1)")
        if not bb.AdaptiveConditioning:
            raise ValueError("FlowDenoiser requires adaptive conditioning in its backbone")
        self.Config_ = c
        self.InputProjection_ = self.RegisterModule("input_projection", OaLinear(c.InputDim, bb.DModel))
        self.TimeEmbedding_ = self.RegisterModule("time_embedding", OaFlowTimeEmbedding(bb.DModel, c.TimeMaxPeriod, c.TimeScale))
        self.ConditionProjection_ = self.RegisterModule("condition_projection", OaLinear(c.ConditionDim, bb.DModel)) if c.ConditionDim > 0 else None
        self.Backbone_ = self.RegisterModule("backbone", OaFlowTransformer(bb))
        self.OutputProjection_ = self.RegisterModule("output_projection", OaLinear(bb.DModel, c.InputDim))
        self.Position_ = self.RegisterParameter("position", F.RandN([bb.SequenceLength, bb.DModel], std=0.02)).Data

    def Forward(self, sample: OaMatrix) -> OaMatrix:
        return self.ForwardConditioned(sample, F.Zeros([sample.Size(0)], torch.float32))

    def ForwardConditioned(self, sample: OaMatrix, time: OaMatrix, condition: Optional[OaMatrix] = None,
                           token_mask: Optional[OaMatrix] = None) -> OaMatrix:
        c, bb = self.Config_, self.Config_.Backbone
        if sample.Rank() != 3 or sample.Size(1) != bb.SequenceLength or sample.Size(2) != c.InputDim:
            raise ValueError("FlowDenoiser expects [B,S,InputDim] samples")
        B, S, D = sample.Size(0), bb.SequenceLength, bb.DModel
        x = self.InputProjection_.Forward(F.Reshape(sample, [B * S, c.InputDim]))
        x = F.Reshape(F.Add(F.Reshape(x, [B, S, D]), F.Reshape(self.Position_, [1, S, D])), [B * S, D])
        ctx = F.Cast(self.TimeEmbedding_.Forward(time), x.Tensor().dtype)
        if condition is not None:
            if self.ConditionProjection_ is None or condition.Rank() != 2 or condition.Size(0) != B or condition.Size(1) != c.ConditionDim:
                raise ValueError("FlowDenoiser condition must be [B,ConditionDim]")
            cond = self.ConditionProjection_.Forward(condition)
            if self.IsTraining() and c.ConditionDropoutP > 0.0:
                keep = F.GreaterEqual(F.Rand([B, 1], cond.Tensor().dtype), F.Full([B, 1], c.ConditionDropoutP, cond.Tensor().dtype))
                cond = F.Mul(cond, keep)
            ctx = F.Add(ctx, cond)
        out = self.Backbone_.ForwardConditioned(x, ctx, token_mask)
        return F.Reshape(self.OutputProjection_.Forward(out), [B, S, c.InputDim])

    def ForwardGuided(self, sample, time, condition, guidance_scale: float, token_mask: Optional[OaMatrix] = None) -> OaMatrix:
        """Classifier-free guidance: uncond + scale * (cond - uncond)."""
        cond = self.ForwardConditioned(sample, time, condition, token_mask)
        uncond = self.ForwardConditioned(sample, time, None, token_mask)
        return F.Add(uncond, F.Scale(F.Sub(cond, uncond), guidance_scale))

    def Config(self) -> OaFlowDenoiserConfig: return self.Config_
    def IsMoe(self) -> bool: return self.Backbone_.IsMoe()
    def Backbone(self) -> OaFlowTransformer: return self.Backbone_
