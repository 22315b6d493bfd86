"""The canonical small-model NLP suite: five architectures x three tokenizers on one 576-byte corpus
(Source/Public/Oa/Ml/NlpSuite.h:11-119, Source/Private/Oa/Ml/NlpSuite.cpp:17-418).

Every recipe shares context 16, width 32, hidden 64, batch 64, 300 steps, seed 20260714, prompt "to be" and 80 generated
source units, so that architectures and tokenizers can be compared on equal terms.  Module names are checkpoint names:
`embed`, `rnn` / `gru` / (`pos_embed`, `block`, `ln_final`) / `mamba3`, `head`.
"""
from __future__ import annotations

import enum
from typing import Optional, Sequence

import torch

from ..core import fn_matrix as F
from ..core.matrix import OaMatrix
from .byte import OaByteEmbedding
from .module import OaModule
from .nn.layers import OaEmbedding, OaLayerNorm, OaLinear, OaTransformerBlock
from .nn.mamba3 import OaMamba3Module
from .nn.moe import OaMoE
from .nn.recurrent import OaGru, OaRnn
from .tokenizer import OaBpeTokenizer


class OaNlpArchitecture(enum.IntEnum):
    Rnn = 0
    Gru = 1
    Transformer = 2
    MoeTransformer = 3
    Mamba3 = 4


class OaNlpTokenizerKind(enum.IntEnum):
    Byte = 0
    Bpe = 1
    Char = 2


OaNlpSuiteContextLength = 16
OaNlpSuiteModelWidth = 32
OaNlpSuiteHiddenWidth = 64
OaNlpSuiteTrainingSteps = 300
OaNlpSuiteBatchSize = 64
OaNlpSuiteRngSeed = 20260714
OaNlpSuiteGenerationPrompt = "to be"
OaNlpSuiteGenerationSourceUnits = 80

_ARCH = {
    OaNlpArchitecture.Rnn: ("rnn", "RNN", "Embedding(32) -> RNN(32x64) -> Linear(vocab)", "nlp_rnn_step"),
    OaNlpArchitecture.Gru: ("gru", "GRU", "Embedding(32) -> GRU(32x64) -> Linear(vocab)", "nlp_gru_step"),
    OaNlpArchitecture.Transformer: ("transformer", "Transformer", "Embedding(32) -> Transformer(FFN=64) -> Linear(vocab)", "nlp_transformer_step"),
    OaNlpArchitecture.MoeTransformer: ("moe", "MoE Transformer", "Embedding(32) -> MoE(E=4,K=2,DFF=16) -> Linear(vocab)", "nlp_moe_step"),
    OaNlpArchitecture.Mamba3: ("mamba3", "Mamba-3", "Embedding(32) -> Mamba-3(state=32) -> Linear(vocab)", "nlp_mamba3_step"),
}
_TOK = {OaNlpTokenizerKind.Byte: ("byte", "Byte", 256), OaNlpTokenizerKind.Bpe: ("bpe", "BPE", 320), OaNlpTokenizerKind.Char: ("char", "Char", 27)}


class OaNlpSuiteRecipe:
    def __init__(self, architecture: OaNlpArchitecture = OaNlpArchitecture.Gru, tokenizer: OaNlpTokenizerKind = OaNlpTokenizerKind.Byte):
        self.Architecture_, self.Tokenizer_ = OaNlpArchitecture(architecture), OaNlpTokenizerKind(tokenizer)

    def Architecture(self): return self.Architecture_
    def Tokenizer(self): return self.Tokenizer_
    def VocabSize(self) -> int: return _TOK[self.Tokenizer_][2]
    def ContextLength(self) -> int: return OaNlpSuiteContextLength
    def ModelWidth(self) -> int: return OaNlpSuiteModelWidth
    def HiddenWidth(self) -> int: return OaNlpSuiteHiddenWidth
    def LearningRate(self) -> float: return 0.003 if self.Architecture_ == OaNlpArchitecture.Mamba3 else 0.01
    def ArchitectureId(self) -> str: return _ARCH[self.Architecture_][0]
    def ArchitectureName(self) -> str: return _ARCH[self.Architecture_][1]
    def ModelDescription(self) -> str: return _ARCH[self.Architecture_][2]
    def TimerName(self) -> str: return _ARCH[self.Architecture_][3]
    def TokenizerId(self) -> str: return _TOK[self.Tokenizer_][0]
    def TokenizerName(self) -> str: return _TOK[self.Tokenizer_][1]


class OaNlpSuiteModel(OaModule):
    def __init__(self, recipe: OaNlpSuiteRecipe):
        super().__init__()
        self.Recipe_ = recipe
        V, D, Hd, S = recipe.VocabSize(), recipe.ModelWidth(), recipe.HiddenWidth(), recipe.ContextLength()
        arch = recipe.Architecture()
        recurrent = arch in (OaNlpArchitecture.Rnn, OaNlpArchitecture.Gru)
        if recipe.Tokenizer() == OaNlpTokenizerKind.Byte and recurrent:
            self.TokenEmbedding = OaByteEmbedding(D)
        else:
            self.TokenEmbedding = OaEmbedding(V, D)
        self.TokenEmbedding.Weight.Data.Tensor().copy_(F.RandN([V, D]).Tensor())        # unit-variance token vectors
        self.RegisterModule("embed", self.TokenEmbedding)
        self.Rnn = self.Gru = self.Transformer = self.FinalNorm = self.PositionEmbedding = self.Mamba3 = None
        head_in = Hd if recurrent else D
        self.Head = OaLinear(head_in, V)
        head_init = F.RandXavier if (arch == OaNlpArchitecture.Gru and recipe.Tokenizer() == OaNlpTokenizerKind.Char) else F.Rand
        if arch != OaNlpArchitecture.Mamba3:
            self.Head.Weight.Data.Tensor().copy_(head_init([V, head_in]).Tensor())
        if arch == OaNlpArchitecture.Rnn:
            self.Rnn = self.RegisterModule("rnn", OaRnn(D, Hd, 1))
        elif arch == OaNlpArchitecture.Gru:
            self.Gru = self.RegisterModule("gru", OaGru(D, Hd, 1))
        elif arch in (OaNlpArchitecture.Transformer, OaNlpArchitecture.MoeTransformer):
            self.PositionEmbedding = self.RegisterModule("pos_embed", OaEmbedding(S, D))
            moe = OaMoE(D, 16, 4, 2) if arch == OaNlpArchitecture.MoeTransformer else None
            self.Transformer = self.RegisterModule("block", OaTransformerBlock(D, Hd, S, 1, 1e-5, moe=moe))
            self.FinalNorm = self.RegisterModule("ln_final", OaLayerNorm(D, 1e-5))
        else:
            self.Mamba3 = self.RegisterModule("mamba3", OaMamba3Module(D, 32, 2, 16, 1, 0.5, False, 4, 0.001, 0.1, 1e-4, 1e-4, True))
        self.RegisterModule("head", self.Head)
        self._hidden: Optional[OaMatrix] = None
        for p in self.AllParameterPtrs():
            p.Data.SetRequiresGrad(True)

    def Recipe(self) -> OaNlpSuiteRecipe:
        return self.Recipe_

    def Forward(self, tokens: OaMatrix) -> OaMatrix:
        """tokens [batch, seq] -> logits [batch*seq, vocab]."""
        r = self.Recipe_
        batch, seq = tokens.Size(0), tokens.Size(1)
        D, Hd, rows = r.ModelWidth(), r.HiddenWidth(), batch * seq
        arch = r.Architecture()
        if arch in (OaNlpArchitecture.Transformer, OaNlpArchitecture.MoeTransformer):
            x = F.Embedding(self.TokenEmbedding.Weight.Data, tokens, self.PositionEmbedding.Weight.Data, seq)
            return self.Head.Forward(self.FinalNorm.Forward(self.Transformer.Forward(x, batch, seq)))
        emb = F.Embedding(self.TokenEmbedding.Weight.Data, tokens, None, seq)
        if arch == OaNlpArchitecture.Rnn:
            return self.Head.Forward(self.Rnn.Forward(emb.Reshape([batch, seq, D])).Reshape([rows, Hd]))
        if arch == OaNlpArchitecture.Gru:
            return self.Head.Forward(self.Gru.Forward(emb.Reshape([batch, seq, D])).Reshape([rows, Hd]))
        mixed = self.Mamba3.Forward(emb.Reshape([batch, seq, D])).Reshape([rows, D])
        return self.Head.Forward(F.Add(mixed, emb))

    # ---- stateful generation (recurrent architectures carry their state; the Transformers re-run the window)
    def SupportsStatefulGeneration(self) -> bool:
        return self.Recipe_.Architecture() in (OaNlpArchitecture.Rnn, OaNlpArchitecture.Gru, OaNlpArchitecture.Mamba3)

    def ResetGenerationState(self, batch: int = 1) -> None:
        arch = self.Recipe_.Architecture()
        if arch == OaNlpArchitecture.Rnn:
            self._hidden = self.Rnn.ZeroState(batch)
        elif arch == OaNlpArchitecture.Gru:
            self._hidden = self.Gru.ZeroState(batch)
        elif arch == OaNlpArchitecture.Mamba3:
            self.Mamba3.ResetState()
        else:
            raise RuntimeError("ResetGenerationState requires an RNN, GRU, or Mamba-3 NLP recipe")

    def ForwardGenerationStep(self, token: OaMatrix) -> OaMatrix:
        if not self.SupportsStatefulGeneration():
            raise RuntimeError("ForwardGenerationStep requires an RNN, GRU, or Mamba-3 NLP recipe")
        if token.Rank() != 2 or token.Size(1) != 1:
            raise ValueError("ForwardGenerationStep expects token ids with shape [batch, 1]")
        batch, D = token.Size(0), self.Recipe_.ModelWidth()
        emb = F.Embedding(self.TokenEmbedding.Weight.Data, token, None, 1).Reshape([batch, D])
        arch = self.Recipe_.Architecture()
        if arch == OaNlpArchitecture.Rnn:
            self._hidden = self.Rnn.Step(emb, self._hidden)
            return self.Head.Forward(self._hidden)
        if arch == OaNlpArchitecture.Gru:
            self._hidden = self.Gru.Step(emb, self._hidden)
            return self.Head.Forward(self._hidden)
        return self.Head.Forward(F.Add(self.Mamba3.Step(emb), emb))


_CORPUS_LINE = ("to be or not to be that is the question whether tis nobler in the mind to suffer the slings and arrows of outrageous "
                "fortune or to take arms against a sea of troubles and by opposing end them ")


class OaNlpSuiteSampler:
    """Deterministic batches from the corpus: sequence b of a batch starts at (cursor + 7 b) mod limit; the cursor advances
    by the batch size."""

    def __init__(self, recipe: OaNlpSuiteRecipe, batch_size: int = OaNlpSuiteBatchSize):
        self.Recipe_, self.BatchSize = recipe, max(1, int(batch_size))
        self.Bpe = OaBpeTokenizer(320)
        if recipe.Tokenizer() == OaNlpTokenizerKind.Bpe:
            self.Bpe.Train(self.Corpus(), 64)
        self.Tokens = self.Encode(self.Corpus())
        self._units = [self._token_source_units(t) for t in range(recipe.VocabSize())]
        self.Cursor, self.LastSourceUnits_ = 0, 0

    @staticmethod
    def Corpus() -> str:
        return _CORPUS_LINE * 3

    def LastSourceUnits(self) -> int:
        return self.LastSourceUnits_

    def Next(self):
        """Returns (input [B, S], target [B, S]) id matrices."""
        S = self.Recipe_.ContextLength()
        limit = len(self.Tokens) - S - 1
        tok = self.Tokens
        inp, tgt = [], []
        self.LastSourceUnits_ = 0
        for b in range(self.BatchSize):
            start = (self.Cursor + b * 7) % limit
            inp += tok[start:start + S]
            row = tok[start + 1:start + S + 1]
            tgt += row
            self.LastSourceUnits_ += sum(self._units[t] for t in row)
        self.Cursor = (self.Cursor + self.BatchSize) % limit
        return self._matrix(inp, self.BatchSize), self._matrix(tgt, self.BatchSize)

    def Encode(self, text: str) -> list:
        kind = self.Recipe_.Tokenizer()
        if kind == OaNlpTokenizerKind.Bpe:
            return self.Bpe.Encode(text)
        if kind == OaNlpTokenizerKind.Char:
            return [ord(c) - 97 if "a" <= c <= "z" else 26 for c in text]
        return list(text.encode("latin-1", errors="replace"))

    def Decode(self, tokens: Sequence[int]) -> str:
        kind = self.Recipe_.Tokenizer()
        if kind == OaNlpTokenizerKind.Bpe:
            return self.Bpe.Decode(tokens)
        if kind == OaNlpTokenizerKind.Char:
            return "".join(chr(97 + t) if 0 <= t < 26 else " " for t in tokens)
        return bytes(int(t) & 0xFF for t in tokens).decode("latin-1")

    def InputMatrix(self, tokens: Sequence[int]) -> OaMatrix:
        S = self.Recipe_.ContextLength()
        return self._matrix(list(tokens), len(tokens) // S)

    def InputStepMatrix(self, token: int) -> OaMatrix:
        return F.FromInt32([int(token)], [1, 1])

    def _token_source_units(self, token: int) -> int:
        if self.Recipe_.Tokenizer() == OaNlpTokenizerKind.Bpe:
            return len(self.Bpe.DecodeBytes([token]))
        return 1

    def _matrix(self, tokens: list, batch: int) -> OaMatrix:
        return F.FromInt32(tokens, [batch, self.Recipe_.ContextLength()])


def OaNlpSuiteGenerate(model: OaNlpSuiteModel, sampler: OaNlpSuiteSampler, prompt: str = OaNlpSuiteGenerationPrompt,
                       source_units: int = OaNlpSuiteGenerationSourceUnits) -> str:
    """Greedy generation until `source_units` source units (bytes / characters) have been produced after the prompt.
    Recurrent recipes carry their state token by token; Transformer recipes re-run the last context window."""
    from . import autograd as AG
    toks = sampler.Encode(prompt)
    S = model.Recipe().ContextLength()
    produced = 0
    with AG.OaGradNo():
        if model.SupportsStatefulGeneration():
            model.ResetGenerationState(1)
            logits = None
            for t in toks:
                logits = model.ForwardGenerationStep(sampler.InputStepMatrix(t))
            while produced < source_units:
                nxt = int(logits.Tensor().float().argmax(-1).reshape(-1)[0])
                toks.append(nxt)
                produced += max(1, sampler._units[nxt])
                logits = model.ForwardGenerationStep(sampler.InputStepMatrix(nxt))
        else:
            while produced < source_units:
                window = toks[-S:]
                ids = F.FromInt32(window, [1, len(window)])
                logits = model.Forward(ids).Tensor().float()
                nxt = int(logits[len(window) - 1].argmax())
                toks.append(nxt)
                produced += max(1, sampler._units[nxt])
    return sampler.Decode(toks)
