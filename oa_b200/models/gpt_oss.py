"""OaGptOssConfig: the architecture contract of the published gpt-oss checkpoints (configuration and validation only, as in
the reference: Extensions/Public/Ml/Nn/GptOss/GptOss.h:10-51, Extensions/Private/Ml/Nn/GptOss/GptOss.cpp).

Grouped-query attention with 64 query / 8 key-value heads of width 64, layers alternating sliding-window (even layers) and
full attention, 32 or 128 experts with top-4 routing and a clamped SwiGLU, YaRN-scaled rotary embeddings, MXFP4 expert
weights.  `Validate()` accepts scaled-down fixtures of the same topology; `FromJson` additionally checks the fields that
identify a published checkpoint.  `YarnInverseFrequencies()` gives the rotary table that the configuration implies.
"""
from __future__ import annotations

import json
import math
from dataclasses import dataclass, replace
from typing import List, Tuple


def _near(a: float, b: float) -> bool:
    return abs(a - b) <= 1e-6 * max(1.0, abs(b))


@dataclass
class OaGptOssConfig:
    VocabSize: int = 201088
    NumLayers: int = 24
    HiddenSize: int = 2880
    IntermediateSize: int = 2880
    NumAttentionHeads: int = 64
    NumKvHeads: int = 8
    HeadDim: int = 64
    NumExperts: int = 32
    ExpertsPerToken: int = 4
    SlidingWindow: int = 128
    OriginalContextLength: int = 4096
    MaxPositionEmbeddings: int = 131072
    RopeTheta: float = 150000.0
    RopeScalingFactor: float = 32.0
    RopeNtkAlpha: float = 1.0      # "beta_slow" in the published JSON
    RopeNtkBeta: float = 32.0      # "beta_fast"
    RmsNormEps: float = 1e-5
    SwiGluAlpha: float = 1.702
    SwiGluLimit: float = 7.0
    PadToken: int = 199999
    EosToken: int = 200002
    AttentionBias: bool = True
    TieWordEmbeddings: bool = False
    MxFp4Experts: bool = True

    @staticmethod
    def Preset20B() -> "OaGptOssConfig":
        return OaGptOssConfig()

    @staticmethod
    def Preset120B() -> "OaGptOssConfig":
        return replace(OaGptOssConfig(), NumLayers=36, NumExperts=128)

    def LayerUsesSlidingAttention(self, layer: int) -> bool:
        return (layer & 1) == 0

    def QueryWidth(self) -> int: return self.NumAttentionHeads * self.HeadDim
    def KvWidth(self) -> int: return self.NumKvHeads * self.HeadDim
    def ExpectedLogicalWeightCount(self) -> int: return 3 + self.NumLayers * 19

    def Validate(self) -> Tuple[bool, str]:
        """(ok, message): topology checks that scaled-down parity fixtures also pass."""
        c = self
        if min(c.VocabSize, c.NumLayers, c.HiddenSize, c.IntermediateSize, c.NumAttentionHeads, c.NumKvHeads, c.HeadDim, c.NumExperts,
               c.ExpertsPerToken, c.SlidingWindow, c.OriginalContextLength) <= 0 or c.ExpertsPerToken > c.NumExperts \
                or c.MaxPositionEmbeddings < c.OriginalContextLength:
            return False, "gpt-oss config: dimensions/counts are inconsistent"
        if c.NumAttentionHeads % c.NumKvHeads != 0:
            return False, "gpt-oss config: attention heads must form integer GQA groups"
        if c.HeadDim % 2 != 0 or c.RopeTheta <= 0 or c.RopeScalingFactor < 1 or c.RopeNtkAlpha <= 0 or c.RopeNtkBeta <= c.RopeNtkAlpha:
            return False, "gpt-oss config: invalid YaRN/RoPE parameters"
        if c.RmsNormEps <= 0 or c.SwiGluAlpha <= 0 or c.SwiGluLimit <= 0:
            return False, "gpt-oss config: invalid normalization/activation parameters"
        if not (0 <= c.PadToken < c.VocabSize and 0 <= c.EosToken < c.VocabSize):
            return False, "gpt-oss config: special token is outside vocabulary"
        if not c.AttentionBias or c.TieWordEmbeddings or not c.MxFp4Experts:
            return False, "gpt-oss config: published bias/embedding/MXFP4 contract changed"
        return True, ""

    @staticmethod
    def FromJson(path: str) -> "OaGptOssConfig":
        """Reads a Hugging Face style config.json; raises ValueError with the failed rule."""
        try:
            with open(path) as f:
                root = json.load(f)
        except (OSError, json.JSONDecodeError) as e:
            raise ValueError(f"gpt-oss config parse failed: {e}") from e
        rope = root.get("rope_scaling") or {}
        out = OaGptOssConfig(
            VocabSize=int(root.get("vocab_size", 0)), NumLayers=int(root.get("num_hidden_layers", 0)), HiddenSize=int(root.get("hidden_size", 0)),
            IntermediateSize=int(root.get("intermediate_size", 0)), NumAttentionHeads=int(root.get("num_attention_heads", 0)),
            NumKvHeads=int(root.get("num_key_value_heads", 0)), HeadDim=int(root.get("head_dim", 0)),
            NumExperts=int(root.get("num_local_experts", 0)),
            ExpertsPerToken=int(root.get("num_experts_per_tok", root.get("experts_per_token", 0))),
            SlidingWindow=int(root.get("sliding_window", 0)), OriginalContextLength=int(root.get("initial_context_length", 0)),
            MaxPositionEmbeddings=int(root.get("max_position_embeddings", 0)), RopeTheta=float(root.get("rope_theta", 0.0)),
            RopeScalingFactor=float(rope.get("factor", 0.0)), RopeNtkAlpha=float(rope.get("beta_slow", 0.0)),
            RopeNtkBeta=float(rope.get("beta_fast", 0.0)), RmsNormEps=float(root.get("rms_norm_eps", 0.0)),
            SwiGluLimit=float(root.get("swiglu_limit", 0.0)), PadToken=int(root.get("pad_token_id", -1)), EosToken=int(root.get("eos_token_id", -1)),
            AttentionBias=bool(root.get("attention_bias", False)), TieWordEmbeddings=bool(root.get("tie_word_embeddings", True)))
        ok, msg = out.Validate()
        if not ok:
            raise ValueError(msg)
        if root.get("model_type", "") != "gpt_oss":
            raise ValueError("gpt-oss config: model_type must be gpt_oss")
        layers = root.get("layer_types")
        if not isinstance(layers, list) or len(layers) != out.NumLayers:
            raise ValueError("gpt-oss config: invalid layer_types count")
        for i, kind in enumerate(layers):
            if kind != ("sliding_attention" if out.LayerUsesSlidingAttention(i) else "full_attention"):
                raise ValueError("gpt-oss config: layer_types must alternate sliding/full from layer zero")
        if (root.get("quantization_config") or {}).get("quant_method", "") != "mxfp4":
            raise ValueError("gpt-oss config: expected MXFP4 experts")
        return out

    def IsPublished20B(self) -> bool:
        p = OaGptOssConfig.Preset20B()
        ints = ("VocabSize", "NumLayers", "HiddenSize", "IntermediateSize", "NumAttentionHeads", "NumKvHeads", "HeadDim", "NumExperts",
                "ExpertsPerToken", "SlidingWindow", "OriginalContextLength", "MaxPositionEmbeddings", "PadToken", "EosToken")
        floats = ("RopeTheta", "RopeScalingFactor", "RopeNtkAlpha", "RopeNtkBeta", "RmsNormEps", "SwiGluLimit")
        return all(getattr(self, n) == getattr(p, n) for n in ints) and all(_near(getattr(self, n), getattr(p, n)) for n in floats)

    def IsPublished120B(self) -> bool:
        return self.NumLayers == 36 and self.NumExperts == 128 and replace(self, NumLayers=24, NumExperts=32).IsPublished20B()

    # ---- derived quantities
    def YarnInverseFrequencies(self) -> Tuple[List[float], float]:
        """(inverse frequencies for the HeadDim/2 rotary pairs, attention scale multiplier).  Pairs whose wavelength fits the
        original context `beta_fast` times keep their frequency, pairs that fit fewer than `beta_slow` times are divided by the
        scaling factor, and the ramp between the two blends linearly; the multiplier is 0.1 ln(factor) + 1."""
        half = self.HeadDim // 2
        base = [self.RopeTheta ** (-2.0 * i / self.HeadDim) for i in range(half)]
        if self.RopeScalingFactor <= 1.0:
            return base, 1.0

        def correction_dim(rotations: float) -> float:
            return self.HeadDim * math.log(self.OriginalContextLength / (rotations * 2 * math.pi)) / (2 * math.log(self.RopeTheta))

        low, high = correction_dim(self.RopeNtkBeta), correction_dim(self.RopeNtkAlpha)
        out = []
        for i, f in enumerate(base):
            ramp = min(max((i - low) / max(high - low, 1e-3), 0.0), 1.0)       # 0: keep (extrapolate), 1: fully interpolated
            out.append(f * (1 - ramp) + (f / self.RopeScalingFactor) * ramp)
        return out, 0.1 * math.log(self.RopeScalingFactor) + 1.0

    def ParameterCount(self) -> int:
        """Logical parameters (embeddings, attention with biases and sinks, router, experts with biases, norms, head)."""
        h, q, kv, e, f = self.HiddenSize, self.QueryWidth(), self.KvWidth(), self.NumExperts, self.IntermediateSize
        attn = h * (q + 2 * kv) + (q + 2 * kv) + q * h + h + self.NumAttentionHeads
        moe = h * e + e + e * (h * 2 * f + 2 * f) + e * (f * h + h)
        return 2 * self.VocabSize * h + h + self.NumLayers * (attn + moe + 2 * h)
