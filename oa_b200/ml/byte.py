"""Byte-level modelling helpers (Source/Public/Oa/Ml/Byte.h:41-116): an embedding over the 256 byte values, the matching
output head, and OaByteEncoder (bytes <-> id matrices, greedy and temperature / nucleus sampling from logits)."""
from __future__ import annotations

from typing import Optional

import torch

from ..core import fn_matrix as F
from ..core.matrix import OaMatrix
from .module import OaModule

OA_BYTE_VOCAB_SIZE = 256


class OaByteEmbedding(OaModule):
    def __init__(self, d_model: int):
        super().__init__()
        self.DModel_ = d_model
        self.Weight = self.RegisterParameter("weight", F.RandN([OA_BYTE_VOCAB_SIZE, d_model]))

    def DModel(self) -> int:
        return self.DModel_

    def Forward(self, byte_ids: OaMatrix) -> OaMatrix:
        """[batch, seq] ids -> [batch, seq, d_model]."""
        out = F.Embedding(self.Weight.Data, byte_ids, None, 0)
        return out.Reshape(list(byte_ids.Tensor().shape) + [self.DModel_])


class OaByteHead(OaModule):
    def __init__(self, d_model: int):
        super().__init__()
        self.DModel_ = d_model
        self.Weight = self.RegisterParameter("weight", F.Rand([OA_BYTE_VOCAB_SIZE, d_model]))
        self.Bias = self.RegisterParameter("bias", F.Zeros([OA_BYTE_VOCAB_SIZE]))

    def Forward(self, hidden: OaMatrix) -> OaMatrix:
        """[..., d_model] -> [..., 256] logits."""
        shape = list(hidden.Tensor().shape)
        y = F.Linear(hidden.Reshape([-1, self.DModel_]) if len(shape) != 2 else hidden, self.Weight.Data, self.Bias.Data)
        return y.Reshape(shape[:-1] + [OA_BYTE_VOCAB_SIZE])


class OaByteEncoder:
    @staticmethod
    def Encode(data) -> OaMatrix:
        b = data.encode("utf-8") if isinstance(data, str) else bytes(data)
        return F.FromInt32(list(b), [len(b)])

    @staticmethod
    def EncodeBatched(data) -> OaMatrix:
        b = data.encode("utf-8") if isinstance(data, str) else bytes(data)
        return F.FromInt32(list(b), [1, len(b)])

    EncodeText = Encode

    @staticmethod
    def EncodeImage(pixels, width: int, height: int, channels: int) -> OaMatrix:
        b = bytes(pixels)
        if len(b) != width * height * channels:
            raise ValueError("pixel buffer does not match width * height * channels")
        return F.FromInt32(list(b), [len(b)])

    @staticmethod
    def EncodeAudio(samples, sample_rate: int = 0, channels: int = 1) -> OaMatrix:
        b = bytes(samples)
        return F.FromInt32(list(b), [len(b)])

    @staticmethod
    def Decode(logits: OaMatrix) -> bytes:
        """Greedy: argmax over the last dimension of [seq, 256] logits."""
        return bytes(int(i) & 0xFF for i in logits.Tensor().float().argmax(-1).reshape(-1).tolist())

    @staticmethod
    def Sample(logits: OaMatrix, temperature: float = 1.0, top_p: float = 0.9, generator: Optional[torch.Generator] = None) -> bytes:
        """Temperature + nucleus sampling, one byte per row of [seq, 256] logits."""
        t = logits.Tensor().float().cpu().reshape(-1, logits.Size(-1))
        if temperature <= 0:
            return OaByteEncoder.Decode(logits)
        probs = torch.softmax(t / temperature, -1)
        sp, si = probs.sort(-1, descending=True)
        keep = (sp.cumsum(-1) - sp) < top_p              # always keeps the most likely byte
        sp = sp * keep
        sp = sp / sp.sum(-1, keepdim=True)
        pick = torch.multinomial(sp, 1, generator=generator)
        return bytes(int(i) & 0xFF for i in si.gather(-1, pick).reshape(-1).tolist())
