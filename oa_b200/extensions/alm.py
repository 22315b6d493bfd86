"""Animation language model: CLIP text encoder, convolutional VQ motion tokenizer, autoregressive Transformer prior,
and the assembled text-to-motion model with one-file deployment.

Parity (paths inside the reference): Extensions/Public/Ml/Nn/Alm/AlmConfig.h (configs), ClipTextAg.h + ClipTextAg.cpp
(text transformer, pooled at the end-of-text row), ClipTokenizer.h, ClipTextWeightAdapter.h (checkpoint name map),
AlmTokenizerAg.h + AlmTokenizerAg.cpp:47-260 (encoder / residual VQ / decoder), AlmPriorAg.h + AlmPriorAg.cpp:18-180
(prefix-conditioned decoder, sampling), AlmAg.h (assembly).  Every layer is one of this package's modules, so the
convolutions run as GEMMs over im2col tiles and the attention through the tiled tensor-core kernel on the GPU.
"""
from __future__ import annotations

import enum
import json
import os
from dataclasses import asdict, dataclass, field
from typing import Dict, List, Optional, Sequence

import torch

from ..core import fn_matrix as F
from ..core.matrix import OaMatrix
from ..core.types import OaStatus, OaStatusCode
from ..ml import autograd as AG
from ..ml.module import OaModule
from ..ml.nn.conv import OaConv1d, OaConvTranspose1d
from ..ml.nn.layers import OaEmbedding, OaLayerNorm, OaLinear, OaMultiHeadAttention, OaRmsNorm, OaTransformerBlock
from ..ml.nn.moe import OaMoE
from ..ml.nn.vq import OaResidualVectorQuantizer, OaResidualVqResult, OaVectorQuantizerConfig


# ------------------------------------------------------------------------------------------ configuration
@dataclass
class OaAlmDatasetConfig:
    DataDir: str = ""
    Split: str = "train"
    Corpus: str = "cmp"          # cmp | humanml3d | kit
    MaxClips: int = 0

    @staticmethod
    def FromEnv() -> "OaAlmDatasetConfig":
        e = os.environ
        return OaAlmDatasetConfig(e.get("OA_ALM_DATA_DIR", ""), e.get("OA_ALM_SPLIT", "train"), e.get("OA_ALM_CORPUS", "cmp"),
                                  int(e.get("OA_ALM_MAX_CLIPS", "0")))


@dataclass
class OaAlmTokenizerConfig:
    InputDim: int = 263
    Width: int = 512
    CodeDim: int = 512
    NumCodes: int = 512
    DownT: int = 2               # temporal down-sampling stages: factor 2^DownT
    Depth: int = 3               # residual blocks per stage
    CommitBeta: float = 0.25
    EmaDecay: float = 0.99
    EmaEps: float = 1e-5
    DeadThresh: float = 2.0
    BatchSize: int = 32
    SeqLen: int = 64
    LearningRate: float = 2e-4
    NumEpochs: int = 2000


class OaAlmFfnType(enum.IntEnum):
    Dense = 0
    Moe = 1
    Hybrid = 2


@dataclass
class OaAlmPriorConfig:
    VocabSize: int = 515
    NumCodes: int = 512
    SomToken: int = 512
    EomToken: int = 513
    PadToken: int = 514
    DModel: int = 384
    NumHeads: int = 1
    NumLayers: int = 6
    DFfn: int = 1536
    TextFeatureDim: int = 0
    FfnType: OaAlmFfnType = OaAlmFfnType.Dense
    MoeNumExperts: int = 4
    MoeExpertsPerToken: int = 2
    MoeEvery: int = 2
    MoeBalanceRate: float = 0.0
    MoeAuxLossAlpha: float = 0.0
    MoeRouterZLossBeta: float = 0.0
    BatchSize: int = 32
    SeqLen: int = 128
    MaxSeqLen: int = 260
    LearningRate: float = 1e-4
    NumEpochs: int = 100
    Temperature: float = 1.0
    TopK: int = 0
    TopP: float = 0.9
    MaxGenLen: int = 256

    def UsesMoe(self, layer: int) -> bool:
        if self.FfnType == OaAlmFfnType.Moe:
            return True
        return self.FfnType == OaAlmFfnType.Hybrid and self.MoeEvery > 0 and (layer + 1) % self.MoeEvery == 0

    def SyncVocab(self, num_codes: int) -> None:
        self.NumCodes, self.VocabSize = num_codes, num_codes + 3
        self.SomToken, self.EomToken, self.PadToken = num_codes, num_codes + 1, num_codes + 2


@dataclass
class OaClipTextConfig:
    VocabSize: int = 49408
    ContextLength: int = 77
    HiddenSize: int = 768
    IntermediateSize: int = 3072
    NumHeads: int = 12
    NumLayers: int = 12
    ProjectionDim: int = 768
    LayerNormEps: float = 1e-5
    QuickGeluAlpha: float = 1.702
    BosToken: int = 49406
    EosToken: int = 49407
    PadToken: int = 49407

    def Validate(self) -> OaStatus:
        if min(self.VocabSize, self.ContextLength, self.HiddenSize, self.IntermediateSize, self.NumHeads, self.NumLayers,
               self.ProjectionDim) <= 0:
            return OaStatus(OaStatusCode.InvalidArgument, "CLIP text dimensions must be positive")
        if self.HiddenSize % self.NumHeads:
            return OaStatus(OaStatusCode.InvalidArgument, "hidden size must be divisible by the head count")
        if not all(0 <= t < self.VocabSize for t in (self.BosToken, self.EosToken, self.PadToken)):
            return OaStatus(OaStatusCode.InvalidArgument, "special tokens must lie inside the vocabulary")
        return OaStatus.Ok()

    @staticmethod
    def ViTL14() -> "OaClipTextConfig":
        return OaClipTextConfig()


# ------------------------------------------------------------------------------------------ CLIP tokenizer
class OaClipTokenizer:
    """Lower-cased byte-pair tokenizer with `</w>` word ends.  With a vocabulary (token -> id) and a merge list it
    reproduces the published CLIP tokenisation; without them it falls back to one token per byte (+ word end) so
    that pipelines can be exercised without the vocabulary files."""

    def __init__(self, vocab: Optional[Dict[str, int]] = None, merges: Optional[Sequence[Sequence[str]]] = None,
                 config: Optional[OaClipTextConfig] = None):
        self.Config = config or OaClipTextConfig()
        self._vocab = dict(vocab) if vocab else None
        self._ranks = {tuple(m): i for i, m in enumerate(merges or ())}

    @staticmethod
    def Load(vocab_json: str, merges_txt: str, config: Optional[OaClipTextConfig] = None) -> "OaClipTokenizer":
        with open(vocab_json, encoding="utf-8") as f:
            vocab = json.load(f)
        with open(merges_txt, encoding="utf-8") as f:
            merges = [tuple(l.split()) for l in f.read().splitlines() if l and not l.startswith("#") and len(l.split()) == 2]
        return OaClipTokenizer(vocab, merges, config)

    def _bpe(self, word: str) -> List[str]:
        parts = list(word[:-1]) + [word[-1] + "</w>"]
        while len(parts) > 1:
            pairs = [(self._ranks.get((a, b), 1 << 30), i) for i, (a, b) in enumerate(zip(parts, parts[1:]))]
            rank, i = min(pairs)
            if rank == 1 << 30:
                break
            parts[i:i + 2] = [parts[i] + parts[i + 1]]
        return parts

    def Encode(self, text: str) -> List[int]:
        """[BOS] tokens [EOS] padded / truncated to the context length."""
        c = self.Config
        ids = [c.BosToken]
        for word in " ".join(text.lower().split()).split(" "):
            if not word:
                continue
            if self._vocab is None:
                ids.extend(b % (c.BosToken) for b in word.encode("utf-8"))
            else:
                ids.extend(self._vocab.get(p, self._vocab.get("<|endoftext|>", c.EosToken)) for p in self._bpe(word))
        ids = ids[:c.ContextLength - 1] + [c.EosToken]
        return ids + [c.PadToken] * (c.ContextLength - len(ids))

    def EncodeBatch(self, texts: Sequence[str]) -> OaMatrix:
        rows = [self.Encode(t) for t in texts]
        return F.FromInt32([t for r in rows for t in r], [len(rows), self.Config.ContextLength])

    def EosRows(self, token_ids: OaMatrix) -> OaMatrix:
        """Flat row index (b * context + position) of the first end-of-text token of every sequence."""
        t = token_ids.Tensor().reshape(-1, self.Config.ContextLength).cpu()
        pos = (t == self.Config.EosToken).int().argmax(dim=1)
        return F.FromInt32((torch.arange(t.shape[0]) * self.Config.ContextLength + pos).tolist(), [t.shape[0]])


# ------------------------------------------------------------------------------------------ CLIP text encoder
class _ClipLayer(OaModule):
    """Pre-norm block with causal attention and a quick-GELU MLP: x * sigmoid(alpha * x)."""

    def __init__(self, cfg: OaClipTextConfig):
        super().__init__()
        self._alpha = cfg.QuickGeluAlpha
        self.Ln1 = self.RegisterModule("layer_norm1", OaLayerNorm(cfg.HiddenSize, cfg.LayerNormEps))
        self.Attn = self.RegisterModule("self_attn", OaMultiHeadAttention(cfg.HiddenSize, cfg.NumHeads, cfg.ContextLength, True, True))
        self.Ln2 = self.RegisterModule("layer_norm2", OaLayerNorm(cfg.HiddenSize, cfg.LayerNormEps))
        self.Fc1 = self.RegisterModule("fc1", OaLinear(cfg.HiddenSize, cfg.IntermediateSize))
        self.Fc2 = self.RegisterModule("fc2", OaLinear(cfg.IntermediateSize, cfg.HiddenSize))

    def Forward(self, x: OaMatrix, batch: int = 1, seq: int = 1) -> OaMatrix:
        x = self.Attn.Forward(self.Ln1.Forward(x), batch, seq, residual=x)
        h = self.Fc1.Forward(self.Ln2.Forward(x))
        h = F.Mul(h, F.Sigmoid(F.Scale(h, self._alpha)))
        return F.Add(x, self.Fc2.Forward(h))


class OaClipTextAg(OaModule):
    def __init__(self, config: Optional[OaClipTextConfig] = None):
        super().__init__()
        self.Config_ = config or OaClipTextConfig.ViTL14()
        st = self.Config_.Validate()
        if not st.IsOk():
            raise ValueError(st.message)
        c = self.Config_
        self.TokenEmbedding_ = self.RegisterModule("token_embedding", OaEmbedding(c.VocabSize, c.HiddenSize))
        self.PositionEmbedding_ = self.RegisterModule("position_embedding", OaEmbedding(c.ContextLength, c.HiddenSize))
        self.Layers_ = [self.RegisterModule(f"layers.{i}", _ClipLayer(c)) for i in range(c.NumLayers)]
        self.FinalLayerNorm_ = self.RegisterModule("final_layer_norm", OaLayerNorm(c.HiddenSize, c.LayerNormEps))
        self.TextProjection_ = self.RegisterModule("text_projection", OaLinear(c.HiddenSize, c.ProjectionDim, False))

    def Config(self) -> OaClipTextConfig: return self.Config_

    def Hidden(self, token_ids: OaMatrix) -> OaMatrix:
        """[B * S, hidden] states after the final layer norm."""
        B, S = token_ids.Size(0), token_ids.Size(1)
        if S > self.Config_.ContextLength:
            raise ValueError("token sequence longer than the context length")
        pos = F.FromInt32(list(range(S)) * B, [B, S])
        x = F.Add(self.TokenEmbedding_.Forward(token_ids), self.PositionEmbedding_.Forward(pos)).Reshape([B * S, self.Config_.HiddenSize])
        for layer in self.Layers_:
            x = layer.Forward(x, B, S)
        return self.FinalLayerNorm_.Forward(x)

    def ForwardTokens(self, token_ids: OaMatrix, flat_eos_rows: OaMatrix) -> OaMatrix:
        """[B, projection] text features: the hidden state at each sequence's end-of-text row, projected."""
        return self.TextProjection_.Forward(F.Gather(self.Hidden(token_ids), flat_eos_rows))

    def Forward(self, token_ids: OaMatrix) -> OaMatrix:
        t = token_ids.Tensor().reshape(token_ids.Size(0), -1).cpu()
        pos = (t == self.Config_.EosToken).int().argmax(dim=1)
        rows = F.FromInt32((torch.arange(t.shape[0]) * t.shape[1] + pos).tolist(), [t.shape[0]])
        return self.ForwardTokens(token_ids, rows)

    def Freeze(self) -> None:
        for p in self.AllParameterPtrs():
            p.Data.SetRequiresGrad(False)
        self.Eval()


def OaClipTextWeightName(source_name: str) -> Optional[str]:
    """Checkpoint tensor name of a published CLIP text model -> parameter name of `OaClipTextAg` (None: not a text
    weight, e.g. the vision tower or the logit scale)."""
    n = source_name
    for prefix in ("text_model.", "transformer.text_model."):
        if n.startswith(prefix):
            n = n[len(prefix):]
    if n.startswith("vision_model.") or n.startswith("visual_projection") or n == "logit_scale" or n.endswith("position_ids"):
        return None
    table = {"embeddings.token_embedding.weight": "token_embedding.weight", "embeddings.position_embedding.weight": "position_embedding.weight",
             "final_layer_norm.weight": "final_layer_norm.weight", "final_layer_norm.bias": "final_layer_norm.bias",
             "text_projection.weight": "text_projection.weight"}
    if n in table:
        return table[n]
    if n.startswith("encoder.layers."):
        rest = n[len("encoder."):]
        return rest.replace(".mlp.fc1.", ".fc1.").replace(".mlp.fc2.", ".fc2.")
    return None


# ------------------------------------------------------------------------------------------ motion tokenizer
class OaAlmTokenizerAg(OaModule):
    """1-D convolutional auto-encoder around a vector quantizer: [B * T, features] motion frames -> T / 2^DownT
    discrete codes per clip and back.  Channel-axis layer norms keep every stage bounded."""

    def __init__(self, config: Optional[OaAlmTokenizerConfig] = None):
        super().__init__()
        self.Config_ = c = config or OaAlmTokenizerConfig()
        W = c.Width
        self.Factor_ = 2 ** c.DownT

        def conv(cin, cout, k, stride, pad, name, dilation=1):
            return self.RegisterModule(name, OaConv1d(cin, cout, k, stride, pad, dilation))

        self.EncIn_ = conv(c.InputDim, W, 3, 1, 1, "enc_in")
        self.EncDown_, self.EncRes_, self.DecRes_, self.DecUp_ = [], [], [], []
        for d in range(c.DownT):
            self.EncDown_.append(conv(W, W, 4, 2, 1, f"enc_down{d}"))
            for q in range(c.Depth):
                self.EncRes_.append(conv(W, W, 3, 1, 3, f"enc_res{d}_{q}_a", 3))
                self.EncRes_.append(conv(W, W, 1, 1, 0, f"enc_res{d}_{q}_b"))
        self.EncOut_ = conv(W, c.CodeDim, 3, 1, 1, "enc_out")
        vq = OaVectorQuantizerConfig(NumCodes=c.NumCodes, CodeDim=c.CodeDim, CommitBeta=c.CommitBeta, EmaDecay=c.EmaDecay,
                                     EmaEps=c.EmaEps, DeadThresh=c.DeadThresh, NormCode=True)
        self.Rvq_ = self.RegisterModule("rvq", OaResidualVectorQuantizer(vq, 1))
        self.DecIn_ = conv(c.CodeDim, W, 3, 1, 1, "dec_in")
        for d in range(c.DownT):
            for q in range(c.Depth):
                self.DecRes_.append(conv(W, W, 3, 1, 3, f"dec_res{d}_{q}_a", 3))
                self.DecRes_.append(conv(W, W, 1, 1, 0, f"dec_res{d}_{q}_b"))
            self.DecUp_.append(self.RegisterModule(f"dec_up{d}", OaConvTranspose1d(W, W, 4, 2, 1)))
        self.DecMid_ = conv(W, W, 3, 1, 1, "dec_mid")
        self.DecOut_ = conv(W, c.InputDim, 3, 1, 1, "dec_out")
        self.EncLn_ = [self.RegisterModule(f"enc_ln{i}", OaLayerNorm(W)) for i in range(1 + c.DownT * (1 + c.Depth))]
        self.DecLn_ = [self.RegisterModule(f"dec_ln{i}", OaLayerNorm(W)) for i in range(1 + c.DownT * (c.Depth + 1) + 1)]

    def Config(self) -> OaAlmTokenizerConfig: return self.Config_
    def DownsampleFactor(self) -> int: return self.Factor_
    def Rvq(self) -> OaResidualVectorQuantizer: return self.Rvq_
    def Forward(self, x: OaMatrix) -> OaMatrix: return OaMatrix()          # driven through Encode / Decode

    @staticmethod
    def _norm(ln: OaLayerNorm, h: OaMatrix, relu: bool) -> OaMatrix:
        p = ln.Parameters()
        fn = F.ChannelNormRelu if relu else F.ChannelNorm
        return fn(h, p[0].Data, p[1].Data, h.Size(0), h.Size(1), h.Size(2), 1e-5)

    @staticmethod
    def _conv(conv: OaConv1d, h: OaMatrix, relu: bool = False) -> OaMatrix:
        p = conv.Parameters()
        fn = F.Conv1dReluGemm if relu else F.Conv1dGemm
        return fn(h, p[0].Data, p[1].Data if len(p) > 1 else None, conv.Stride, conv.Padding, conv.Dilation)

    def _res_stack(self, convs: Sequence[OaConv1d], lns: Sequence[OaLayerNorm], cursor: int, h: OaMatrix):
        for q in range(0, len(convs) - 1, 2):
            t = self._conv(convs[q], self._norm(lns[cursor], h, True))
            cursor += 1
            h = F.Add(h, self._conv(convs[q + 1], t, True))
        return h, cursor

    def Encode(self, x: OaMatrix, batch: int, seq_len: int) -> OaMatrix:
        """[B * T, InputDim] -> unit-RMS latents [B * T / factor, CodeDim]."""
        c = self.Config_
        if seq_len % self.Factor_:
            raise ValueError("sequence length must be a multiple of the down-sampling factor")
        h = F.Transpose(x.Reshape([batch, seq_len, c.InputDim]), 1, 2)
        lnc, res = 0, 0
        h = self._norm(self.EncLn_[lnc], self._conv(self.EncIn_, h), True); lnc += 1
        for d in range(c.DownT):
            h = self._norm(self.EncLn_[lnc], self._conv(self.EncDown_[d], h), True); lnc += 1
            h, lnc = self._res_stack(self.EncRes_[res:res + 2 * c.Depth], self.EncLn_, lnc, h)
            res += 2 * c.Depth
        z = F.Transpose(self._conv(self.EncOut_, h), 1, 2).Reshape([batch * (seq_len // self.Factor_), c.CodeDim])
        return F.RmsNorm(z, F.Ones([c.CodeDim], z.Tensor().dtype), 1e-5)

    def Quantize(self, ze: OaMatrix) -> OaResidualVqResult: return self.Rvq_.Quantize(ze)
    def EmaUpdate(self, result: OaResidualVqResult) -> None: self.Rvq_.EmaUpdate(result)
    def Seed(self, latents: OaMatrix) -> None: self.Rvq_.Seed(latents)

    def Decode(self, zq: OaMatrix, batch: int, tok_len: int) -> OaMatrix:
        """[B * tokens, CodeDim] -> [B * tokens * factor, InputDim]."""
        c = self.Config_
        h = F.Transpose(zq.Reshape([batch, tok_len, c.CodeDim]), 1, 2)
        lnc, res = 0, 0
        h = self._norm(self.DecLn_[lnc], self._conv(self.DecIn_, h), True); lnc += 1
        for d in range(c.DownT):
            h, lnc = self._res_stack(self.DecRes_[res:res + 2 * c.Depth], self.DecLn_, lnc, h)
            res += 2 * c.Depth
            h = self._norm(self.DecLn_[lnc], self.DecUp_[d].Forward(h), False); lnc += 1
        h = self._norm(self.DecLn_[lnc], self._conv(self.DecMid_, h), True)
        o = F.Transpose(self._conv(self.DecOut_, h), 1, 2)
        return o.Reshape([batch * tok_len * self.Factor_, c.InputDim])

    def Tokenize(self, x: OaMatrix, batch: int, seq_len: int) -> List[OaMatrix]:
        return self.Rvq_.Quantize(self.Encode(x, batch, seq_len)).Idx

    def Detokenize(self, idx: Sequence[OaMatrix], batch: int, tok_len: int) -> OaMatrix:
        return self.Decode(self.Rvq_.Lookup(idx), batch, tok_len)

    def ReconstructionLoss(self, x: OaMatrix, batch: int, seq_len: int):
        """(loss = mean squared error + commitment, quantizer result) of one training window."""
        from ..ml import fn_loss as L
        res = self.Quantize(self.Encode(x, batch, seq_len))
        recon = self.Decode(res.Quantized, batch, seq_len // self.Factor_)
        return F.Add(L.Mse(recon, x), res.CommitLoss), res


# ------------------------------------------------------------------------------------------ prior
class OaAlmPriorAg(OaModule):
    """Decoder-only Transformer over motion codes [SOM] c1 .. cn [EOM]; an optional text feature is projected and
    prepended as one prefix position."""

    def __init__(self, config: Optional[OaAlmPriorConfig] = None):
        super().__init__()
        self.Config_ = c = config or OaAlmPriorConfig()
        if c.DModel <= 0 or c.NumHeads <= 0 or c.DModel % c.NumHeads or c.DFfn <= 0 or c.NumLayers <= 0 or c.SeqLen <= 0 \
                or c.MaxSeqLen <= 0 or c.SeqLen > c.MaxSeqLen:
            raise ValueError("prior dimensions must be positive, DModel divisible by NumHeads, SeqLen <= MaxSeqLen")
        if c.FfnType != OaAlmFfnType.Dense and (c.MoeNumExperts <= 0 or c.MoeExpertsPerToken <= 0):
            raise ValueError("MoE expert counts must be positive")
        if c.FfnType == OaAlmFfnType.Hybrid and c.MoeEvery <= 0:
            raise ValueError("hybrid MoE cadence must be positive")
        if c.TextFeatureDim < 0:
            raise ValueError("text feature dimension cannot be negative")
        self.TokenEmbed_ = OaEmbedding(c.VocabSize, c.DModel)
        self.TextProjection_ = self.RegisterModule("text_projection", OaLinear(c.TextFeatureDim, c.DModel)) if c.TextFeatureDim > 0 else None
        self.PosEmbed_ = OaEmbedding(c.MaxSeqLen, c.DModel)
        self.Layers_: List[OaTransformerBlock] = []
        for i in range(c.NumLayers):
            moe = None
            if c.UsesMoe(i):
                moe = OaMoE(c.DModel, c.DFfn, c.MoeNumExperts, c.MoeExpertsPerToken, 1e-5)
                moe.SetAuxLossAlpha(c.MoeAuxLossAlpha)
                moe.SetZLossBeta(c.MoeRouterZLossBeta)
            self.Layers_.append(self.RegisterModule(f"layer{i}", OaTransformerBlock(c.DModel, c.DFfn, c.SeqLen, c.NumHeads, 1e-5, moe=moe)))
        self.FinalNorm_ = OaRmsNorm(c.DModel)
        self.OutputHead_ = OaLinear(c.DModel, c.VocabSize, False)
        self.RegisterModule("token_embed", self.TokenEmbed_)
        self.RegisterModule("pos_embed", self.PosEmbed_)
        self.RegisterModule("final_norm", self.FinalNorm_)
        self.RegisterModule("output_head", self.OutputHead_)

    def GetConfig(self) -> OaAlmPriorConfig: return self.Config_

    def _forward(self, token_ids: OaMatrix, text: Optional[OaMatrix]) -> OaMatrix:
        c = self.Config_
        B, T = token_ids.Size(0), token_ids.Size(1)
        prefix = 1 if text is not None else 0
        total = T + prefix
        if B <= 0 or T <= 0 or total > c.MaxSeqLen:
            raise ValueError("input must be non-empty and fit the maximum sequence length")
        emb = self.TokenEmbed_.Forward(token_ids).Reshape([B, T, c.DModel])
        if text is not None:
            if self.TextProjection_ is None or text.Rank() != 2 or text.Size(0) != B or text.Size(1) != c.TextFeatureDim:
                raise ValueError("text features must be [B, TextFeatureDim] and the prior built with TextFeatureDim > 0")
            emb = F.Concat([self.TextProjection_.Forward(text).Reshape([B, 1, c.DModel]), emb], 1)
        pos = F.FromInt32(list(range(total)) * B, [B, total])
        x = F.Add(emb, self.PosEmbed_.Forward(pos).Reshape([B, total, c.DModel])).Reshape([B * total, c.DModel])
        for layer in self.Layers_:
            layer.SetSeqLen(total)
            x = layer.Forward(x, B, total)
        x = self.FinalNorm_.Forward(x)
        if prefix:
            x = F.Slice(x.Reshape([B, total, c.DModel]), 1, 1, total).Reshape([B * T, c.DModel])
        return self.OutputHead_.Forward(x).Reshape([B, T * c.VocabSize])

    def Forward(self, token_ids: OaMatrix) -> OaMatrix:
        """[B, T] ids -> [B, T * vocab] logits."""
        return self._forward(token_ids, None)

    def ForwardConditioned(self, token_ids: OaMatrix, text_features: OaMatrix) -> OaMatrix:
        return self._forward(token_ids, text_features)

    def MoeAuxLoss(self) -> OaMatrix:
        total = None
        for l in self.Layers_:
            if l.Moe is not None and getattr(l.Moe, "LastAuxLoss", None) is not None:
                total = l.Moe.LastAuxLoss if total is None else F.Add(total, l.Moe.LastAuxLoss)
        return total if total is not None else F.Zeros([1])

    def _generate(self, text: Optional[OaMatrix], batch: int, temperature: float, top_k: int, top_p: float, max_len: int, seed: int) -> OaMatrix:
        c = self.Config_
        max_len = min(max_len, c.MaxSeqLen - (1 if text is not None else 0) - 1)
        V = c.VocabSize
        toks = torch.full((batch, 1), c.SomToken, dtype=torch.int32)
        done = torch.zeros(batch, dtype=torch.bool)
        with AG.OaGradNo():
            for step in range(max_len):
                ids = F.FromInt32(toks.reshape(-1).tolist(), list(toks.shape))
                logits = self._forward(ids, text).Tensor().float().reshape(batch, toks.shape[1], V)[:, -1].clone()
                logits[:, c.SomToken] = float("-inf")
                logits[:, c.PadToken] = float("-inf")
                if temperature <= 0:
                    nxt = logits.argmax(-1).to(torch.int32).cpu()
                else:
                    nxt = F.SampleLogits(OaMatrix(logits), temperature, top_k, top_p, seed + step).Tensor().reshape(-1).to(torch.int32).cpu()
                nxt = torch.where(done, torch.full_like(nxt, c.PadToken), nxt)
                toks = torch.cat([toks, nxt[:, None]], dim=1)
                done |= nxt == c.EomToken
                if bool(done.all()):
                    break
        return F.FromInt32(toks.reshape(-1).tolist(), list(toks.shape))

    def Generate(self, batch_size: int, temperature: float = 1.0, top_k: int = 0, top_p: float = 0.9, max_len: int = 256,
                 seed: int = 0) -> OaMatrix:
        """[B, <= max_len + 1] ids starting with [SOM]; rows that ended are padded with [PAD]."""
        return self._generate(None, batch_size, temperature, top_k, top_p, max_len, seed)

    def GenerateConditioned(self, text_features: OaMatrix, temperature: float = 1.0, top_k: int = 0, top_p: float = 0.9,
                            max_len: int = 256, seed: int = 0) -> OaMatrix:
        return self._generate(text_features, text_features.Size(0), temperature, top_k, top_p, max_len, seed)

    def DecodeToMotion(self, token_ids: OaMatrix, tokenizer: OaAlmTokenizerAg) -> List[OaMatrix]:
        """One [frames, InputDim] motion per row: the codes between [SOM] and the first [EOM] / [PAD], detokenized."""
        c, out = self.Config_, []
        for row in token_ids.Tensor().reshape(token_ids.Size(0), -1).cpu().tolist():
            codes = []
            for t in row:
                if t == c.SomToken:
                    continue
                if t >= c.NumCodes:
                    break
                codes.append(t)
            if not codes:
                out.append(OaMatrix())
                continue
            with AG.OaGradNo():
                out.append(tokenizer.Detokenize([F.FromInt32(codes, [len(codes)])], 1, len(codes)))
        return out


# ------------------------------------------------------------------------------------------ assembled model
class OaAlmAg(OaModule):
    """Text -> motion: frozen CLIP text features condition the prior, whose codes the tokenizer decodes.  `Save` writes
    all three parts and their configurations into one `.oam` file."""

    def __init__(self, tokenizer: OaAlmTokenizerAg, prior: OaAlmPriorAg, text: Optional[OaClipTextAg] = None,
                 clip_tokenizer: Optional[OaClipTokenizer] = None):
        super().__init__()
        if prior.GetConfig().NumCodes != tokenizer.Config().NumCodes:
            raise ValueError("prior and tokenizer disagree on the number of motion codes")
        if text is not None and prior.GetConfig().TextFeatureDim != text.Config().ProjectionDim:
            raise ValueError("prior text feature dimension must equal the text encoder's projection dimension")
        self.Tokenizer = self.RegisterModule("tokenizer", tokenizer)
        self.Prior = self.RegisterModule("prior", prior)
        self.Text = self.RegisterModule("text", text) if text is not None else None
        self.ClipTokenizer = clip_tokenizer or (OaClipTokenizer(config=text.Config()) if text is not None else None)

    def Forward(self, token_ids: OaMatrix) -> OaMatrix:
        return self.Prior.Forward(token_ids)

    def OamConfig(self) -> dict:
        cfg = {"tokenizer": asdict(self.Tokenizer.Config()), "prior": {k: int(v) if isinstance(v, enum.Enum) else v
                                                                      for k, v in asdict(self.Prior.GetConfig()).items()}}
        if self.Text is not None:
            cfg["text"] = asdict(self.Text.Config())
        return {"Architecture": "OaAlmAg", "DModel": self.Prior.GetConfig().DModel, "NLayers": self.Prior.GetConfig().NumLayers,
                "DVocab": self.Prior.GetConfig().VocabSize, "ArchConfig": json.dumps(cfg).encode()}

    @staticmethod
    def FromArchConfig(blob: bytes) -> "OaAlmAg":
        cfg = json.loads(bytes(blob).decode())
        prior_cfg = OaAlmPriorConfig(**{**cfg["prior"], "FfnType": OaAlmFfnType(cfg["prior"]["FfnType"])})
        text = OaClipTextAg(OaClipTextConfig(**cfg["text"])) if "text" in cfg else None
        return OaAlmAg(OaAlmTokenizerAg(OaAlmTokenizerConfig(**cfg["tokenizer"])), OaAlmPriorAg(prior_cfg), text)

    @staticmethod
    def LoadOam(path: str) -> "OaAlmAg":
        from ..io.oam import OamModel
        oam, st = OamModel.Load(str(path))
        if oam is None:
            raise ValueError(st.message)
        cfg = oam.GetConfig()
        if cfg["Architecture"] != "OaAlmAg":
            raise ValueError(f"{path} holds a '{cfg['Architecture']}' model")
        model = OaAlmAg.FromArchConfig(cfg["ArchConfig"])
        st = model.LoadFrom(oam)
        if not st.IsOk():
            raise ValueError(st.message)
        return model

    def TextFeatures(self, prompts: Sequence[str]) -> OaMatrix:
        if self.Text is None:
            raise ValueError("the model was assembled without a text encoder")
        ids = self.ClipTokenizer.EncodeBatch(prompts)
        with AG.OaGradNo():
            return self.Text.ForwardTokens(ids, self.ClipTokenizer.EosRows(ids))

    def Generate(self, prompts: Sequence[str], temperature: float = 1.0, top_k: int = 0, top_p: float = 0.9, max_len: int = 64,
                 seed: int = 0) -> List[OaMatrix]:
        """One [frames, features] motion per prompt."""
        toks = self.Prior.GenerateConditioned(self.TextFeatures(prompts), temperature, top_k, top_p, max_len, seed)
        return self.Prior.DecodeToMotion(toks, self.Tokenizer)
