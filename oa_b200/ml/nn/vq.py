"""Vector quantisation: VqAssign / VqEmaUpdate matrix functions and the OaVectorQuantizer / OaResidualVectorQuantizer modules.

Reference: Source/Public/Oa/Ml/FnMatrix.h:223-255 (VqAssign, Detach, VqEmaUpdate) and Source/Public/Oa/Ml/Nn/Vq/Vq.h with
Source/Private/Oa/Ml/Nn/Vq/Vq.cpp.  The codebook is not a gradient parameter: it follows the encoder latents by EMA and is
kept in persistent module buffers (codebook, embed_sum, cluster_size) so it checkpoints with the model.  The assignment
is a GEMM (z . e_k for all codes) followed by one argmin + gather kernel; everything stays on the device.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional, Sequence

import torch

from ... import _native as N
from ...core import fn_matrix as F
from ...core.matrix import OaMatrix
from ...ops import kernels as K
from ...runtime import engine as RT
from ..module import OaModule


@dataclass
class OaVqAssignResult:
    Idx: OaMatrix      # [N] int32 nearest code per row
    Zq: OaMatrix       # [N, D] the winning code per row


def VqAssign(ze: OaMatrix, codebook: OaMatrix) -> OaVqAssignResult:
    """Per-row argmin_k |z - e_k|^2 (lowest index on ties) and the gathered code.  Not differentiable."""
    F._ctx_add("VqAssign")
    z, e = F._c(ze.Tensor().detach()).float(), F._c(codebook.Tensor()).float()
    n, d = z.shape
    kc = e.shape[0]
    if not z.is_cuda:
        dist = (e * e).sum(1)[None, :] - 2.0 * (z @ e.t())
        idx = dist.argmin(1).to(torch.int32)
        return OaVqAssignResult(OaMatrix(idx), OaMatrix(e[idx.long()].to(ze.Tensor().dtype)))
    lib, st = N.require(), N.stream()
    dot = K.gemm(z, e)                                              # [N, K] fp32
    enorm = torch.empty(kc, dtype=torch.float32, device=z.device)
    idx = torch.empty(n, dtype=torch.int32, device=z.device)
    zq = torch.empty(n, d, dtype=torch.float32, device=z.device)
    K._launch(lib.oa_vq_code_norm(e.data_ptr(), enorm.data_ptr(), kc, d, st), "oa_vq_code_norm")
    K._launch(lib.oa_vq_argmin_gather(dot.data_ptr(), enorm.data_ptr(), e.data_ptr(), idx.data_ptr(), zq.data_ptr(), n, kc, d, st),
              "oa_vq_argmin_gather")
    return OaVqAssignResult(OaMatrix(idx), OaMatrix(zq.to(ze.Tensor().dtype)))


def _revival_row(k: int, seed: int, n: int) -> int:
    h = (((k + 1) * 2654435761) ^ (seed * 2246822519) ^ (seed >> 15)) & 0xFFFFFFFF
    h ^= h >> 13
    h = (h * 3266489917) & 0xFFFFFFFF
    h ^= h >> 16
    return h % n


def VqEmaUpdate(ze: OaMatrix, idx: OaMatrix, embed_sum: OaMatrix, cluster_size: OaMatrix, codebook: OaMatrix, decay: float, eps: float,
                dead_threshold: float, seed: int, normalize: bool) -> None:
    """EMA cluster sizes / sums, codebook = sum / max(size, eps), optional unit-RMS rescale, dead-code revival from the
    encoder row hash(code, seed) mod N.  Mutates embed_sum, cluster_size and codebook in place (fp32 buffers)."""
    F._ctx_add("VqEmaUpdate")
    z, ix = F._c(ze.Tensor().detach()).float(), F._c(idx.Tensor())
    es, cs, cb = embed_sum.Tensor(), cluster_size.Tensor(), codebook.Tensor()
    n, d = z.shape
    kc = cb.shape[0]
    assert es.dtype == cs.dtype == cb.dtype == torch.float32 and es.is_contiguous() and cb.is_contiguous()
    if z.is_cuda:
        lib = N.require()
        K._launch(lib.oa_vq_ema_update(z.data_ptr(), ix.data_ptr(), es.data_ptr(), cs.data_ptr(), cb.data_ptr(), n, d, kc, float(decay),
                                       float(eps), float(dead_threshold), int(seed) & 0xFFFFFFFF, int(normalize), N.stream()),
                  "oa_vq_ema_update")
        return
    onehot = torch.zeros(n, kc).scatter_(1, ix.long()[:, None], 1.0)
    nk = decay * cs + (1 - decay) * onehot.sum(0)
    mk = decay * es + (1 - decay) * (onehot.t() @ z)
    ek = mk / nk.clamp(min=eps)[:, None]
    if normalize:
        rms = ek.square().mean(1).sqrt()
        ek = torch.where((rms > eps)[:, None], ek / rms.clamp(min=1e-30)[:, None], ek)
    dead = nk < dead_threshold
    for k in dead.nonzero().flatten().tolist():
        row = z[_revival_row(k, int(seed) & 0xFFFFFFFF, n)]
        ek[k], mk[k], nk[k] = row, row, 1.0
    es.copy_(mk)
    cs.copy_(nk)
    cb.copy_(ek)


@dataclass
class OaVectorQuantizerConfig:
    NumCodes: int = 256
    CodeDim: int = 64
    CommitBeta: float = 0.25
    EmaDecay: float = 0.99
    EmaEps: float = 1e-5
    DeadThresh: float = 1.0
    NormCode: bool = False


@dataclass
class OaVqResult:
    Quantized: OaMatrix       # [N, D] straight-through: z_e + Detach(z_q - z_e)
    Idx: OaMatrix             # [N] int32
    CommitLoss: OaMatrix      # scalar beta * MSE(z_e, sg z_q)


def _commit(ze: OaMatrix, zq: OaMatrix, beta: float) -> OaMatrix:
    d = F.Sub(ze, zq)
    sq = F.Mul(d, d)
    return F.Scale(F.Scale(F.Sum(sq), 1.0 / sq.NumElements()), beta)


class OaVectorQuantizer(OaModule):
    def __init__(self, config: Optional[OaVectorQuantizerConfig] = None):
        super().__init__()
        self.Config_ = config or OaVectorQuantizerConfig()
        Kc, D = self.Config_.NumCodes, self.Config_.CodeDim
        self.Codebook_ = F.RandGlorotUniform([Kc, D], torch.float32)
        self.EmbedSum_ = OaMatrix(self.Codebook_.Tensor().clone())
        self.ClusterSize_ = F.Ones([Kc], torch.float32)
        self.RegisterBuffer("codebook", self.Codebook_)
        self.RegisterBuffer("embed_sum", self.EmbedSum_)
        self.RegisterBuffer("cluster_size", self.ClusterSize_)
        self.EmaStep_ = 0

    def Quantize(self, ze: OaMatrix) -> OaVqResult:
        vq = VqAssign(ze, self.Codebook_)
        quantized = F.Add(ze, F.Detach(F.Sub(vq.Zq, F.Detach(ze))))
        return OaVqResult(quantized, vq.Idx, _commit(ze, vq.Zq, self.Config_.CommitBeta))

    def Forward(self, ze: OaMatrix) -> OaMatrix:
        return self.Quantize(ze).Quantized

    def EmaUpdate(self, ze: OaMatrix, idx: OaMatrix) -> None:
        """Call once per step after the optimizer step with this step's z_e and the indices Quantize returned."""
        c = self.Config_
        VqEmaUpdate(ze, idx, self.EmbedSum_, self.ClusterSize_, self.Codebook_, c.EmaDecay, c.EmaEps, c.DeadThresh, self.EmaStep_, c.NormCode)
        self.EmaStep_ += 1

    def Lookup(self, idx: OaMatrix) -> OaMatrix:
        return F.Gather(self.Codebook_, idx)

    def Seed(self, latents: OaMatrix) -> None:
        """Data-dependent init from the K highest-norm rows of `latents` ([>= K, D]); written in place so the registered
        buffers stay the live state."""
        Kc = self.Config_.NumCodes
        t = latents.Tensor().detach().float()
        if t.shape[0] < Kc:
            raise ValueError("VQ seed needs at least NumCodes latent rows")
        F._ctx_add("VqSeed")
        norms = (t * t).sum(1)
        top = torch.sort(norms, descending=True, stable=True).indices[:Kc]
        seeds = t[top]
        self.Codebook_.Tensor().copy_(seeds)
        self.EmbedSum_.Tensor().copy_(seeds)
        self.ClusterSize_.Tensor().fill_(1.0)
        ctx = RT.OaContext.GetDefault()
        ctx.Execute()
        ctx.Sync()

    def Codebook(self) -> OaMatrix: return self.Codebook_
    def Config(self) -> OaVectorQuantizerConfig: return self.Config_


@dataclass
class OaResidualVqResult:
    Quantized: OaMatrix
    Idx: List[OaMatrix] = field(default_factory=list)          # per level [N] int32 tokens
    Residuals: List[OaMatrix] = field(default_factory=list)    # per level input residual (kept for the EMA update)
    CommitLoss: Optional[OaMatrix] = None


class OaResidualVectorQuantizer(OaModule):
    """Q stacked quantizers: level q quantizes what levels 0..q-1 left; the output is the sum of all levels' codes."""

    def __init__(self, config: OaVectorQuantizerConfig, num_levels: int):
        super().__init__()
        if num_levels < 1:
            raise ValueError("RVQ needs at least one level")
        self.Config_ = config
        self.Levels_ = [self.RegisterModule(f"level{q}", OaVectorQuantizer(config)) for q in range(num_levels)]

    def Quantize(self, ze: OaMatrix) -> OaResidualVqResult:
        residual, total = F.Detach(ze), None
        idxs, residuals = [], []
        for lvl in self.Levels_:
            a = VqAssign(residual, lvl.Codebook())
            residuals.append(residual)
            idxs.append(a.Idx)
            total = a.Zq if total is None else F.Add(total, a.Zq)
            residual = F.Sub(residual, a.Zq)
        quantized = F.Add(ze, F.Detach(F.Sub(total, F.Detach(ze))))
        return OaResidualVqResult(quantized, idxs, residuals, _commit(ze, total, self.Config_.CommitBeta))

    def Forward(self, ze: OaMatrix) -> OaMatrix:
        return self.Quantize(ze).Quantized

    def EmaUpdate(self, result: OaResidualVqResult) -> None:
        for lvl, r, i in zip(self.Levels_, result.Residuals, result.Idx):
            lvl.EmaUpdate(r, i)

    def Lookup(self, idx: Sequence[OaMatrix]) -> OaMatrix:
        if not 1 <= len(idx) <= len(self.Levels_):
            raise ValueError("RVQ Lookup needs between one and NumLevels levels of token ids")
        total = self.Levels_[0].Lookup(idx[0])
        for q in range(1, len(idx)):
            total = F.Add(total, self.Levels_[q].Lookup(idx[q]))
        return total

    def Seed(self, latents: OaMatrix) -> None:
        residual = F.Detach(latents)
        for lvl in self.Levels_:
            lvl.Seed(residual)
            residual = F.Sub(residual, VqAssign(residual, lvl.Codebook()).Zq)

    def NumLevels(self) -> int: return len(self.Levels_)
    def Level(self, q: int) -> OaVectorQuantizer: return self.Levels_[q]
