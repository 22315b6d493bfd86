"""Tensor-parallel decoder-only Transformer (RMSNorm, RoPE, SwiGLU or GELU FFN, no biases) over parallel/tp.py.

Rank r keeps heads [r*H/W, (r+1)*H/W) of every attention layer, columns [r*F/W, (r+1)*F/W) of every FFN and rows
[r*V/W, (r+1)*V/W) of the vocabulary head; norm weights and the embedding table are replicated and their gradients are
summed over the group after the backward pass.  Activations between layers are sharded by rows (sequence parallel), so
norms and residual adds run on 1/W of the tokens.  The model can be cut out of a full OaGptModel (`FromFull`) and owns
the gradient-accumulation loop the 7B-class configuration needs (micro-batch 1 x N accumulation steps).
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist

from ..core import fn_matrix as F
from ..core.matrix import OaMatrix
from ..ml.module import OaModule
from ..ml.nn.layers import OaRmsNorm
from ..models.gpt import OaGptConfig, OaGptModel
from . import tp as TP
from .mesh import OaDeviceMesh


class OaTpBlock(OaModule):
    def __init__(self, cfg: OaGptConfig, arena: TP.OaTpArena, rows: int, full_block=None):
        super().__init__()
        m = arena.mesh
        W, r = m.world, m.rank
        D, Fd, H = cfg.DModel, cfg.DFf, cfg.NHeads
        assert H % W == 0 and Fd % W == 0 and cfg.Norm == "rms" and not cfg.Bias and cfg.RopeTheta > 0
        self.Cfg, self.HeadsLocal, self.HeadDim = cfg, H // W, D // H
        Dl, Fl = D // W, Fd // W
        self.Gated = cfg.Ffn == "swiglu"
        self.LnAttn = self.RegisterModule("ln_attn", OaRmsNorm(D, cfg.Eps))
        self.LnFfn = self.RegisterModule("ln_ffn", OaRmsNorm(D, cfg.Eps))
        std = cfg.InitStd or 0.02
        mk = lambda shape: F.RandN(list(shape), std=std)
        self.Qkv = self.RegisterParameter("qkv.weight", mk((3 * Dl, D)))
        self.Out = self.RegisterParameter("out_proj.weight", mk((D, Dl)))
        self.Up = self.RegisterParameter("up.weight", mk(((2 if self.Gated else 1) * Fl, D)))
        self.Down = self.RegisterParameter("down.weight", mk((D, Fl)))
        if full_block is not None:
            self._cut(full_block, r, Dl, Fl)
        # call sites: forward all-gather / reduce-scatter and their backward mirrors
        self.s_qkv, self.s_qkv_b = TP.OaTpAgSite(arena, rows, D), TP.OaTpRsSite(arena, rows, D)
        self.s_out, self.s_out_b = TP.OaTpRsSite(arena, rows, D), TP.OaTpAgSite(arena, rows, D)
        self.s_up, self.s_up_b = TP.OaTpAgSite(arena, rows, D), TP.OaTpRsSite(arena, rows, D)
        self.s_down, self.s_down_b = TP.OaTpRsSite(arena, rows, D), TP.OaTpAgSite(arena, rows, D)

    def _cut(self, fb, r: int, Dl: int, Fl: int) -> None:
        a = fb.Attention
        sl = slice(r * Dl, (r + 1) * Dl)
        self.Qkv.Data.Tensor().copy_(torch.cat([a.QProj.Weight.Tensor()[sl], a.KProj.Weight.Tensor()[sl], a.VProj.Weight.Tensor()[sl]], 0))
        self.Out.Data.Tensor().copy_(a.OutProj.Weight.Tensor()[:, sl])
        fs = slice(r * Fl, (r + 1) * Fl)
        if self.Gated:
            self.Up.Data.Tensor().copy_(torch.cat([fb.Ffn.Gate.Weight.Tensor()[fs], fb.Ffn.Up.Weight.Tensor()[fs]], 0))
            self.Down.Data.Tensor().copy_(fb.Ffn.Down.Weight.Tensor()[:, fs])
            self.LnFfn.Weight.Data.Tensor().copy_(fb.Ffn.Norm.Weight.Tensor())
        else:
            self.Up.Data.Tensor().copy_(fb.Ffn1.Weight.Tensor()[fs])
            self.Down.Data.Tensor().copy_(fb.Ffn2.Weight.Tensor()[:, fs])
            self.LnFfn.Weight.Data.Tensor().copy_(fb.LnFfn.Weight.Tensor())
        self.LnAttn.Weight.Data.Tensor().copy_(fb.LnAttn.Weight.Tensor())

    def Forward(self, x: OaMatrix, batch: int, seq: int) -> OaMatrix:
        """x [rows / W, D] (this rank's row shard) -> same shape."""
        h = self.LnAttn.Forward(x)
        qkv = TP.ColumnParallelLinear(h, self.Qkv.Data, self.s_qkv, self.s_qkv_b, "TpQkv")
        attn = F.FlashAttentionPacked(qkv, batch, seq, self.HeadsLocal, self.HeadDim, causal=True, rope_theta=self.Cfg.RopeTheta, consume_input=True)
        x = TP.RowParallelLinear(attn, self.Out.Data, self.s_out, self.s_out_b, residual=x, name="TpAttnOut")
        h = self.LnFfn.Forward(x)
        up = TP.ColumnParallelLinear(h, self.Up.Data, self.s_up, self.s_up_b, "TpFfnUp")
        act = F.Swiglu(up) if self.Gated else F.Gelu(up)
        return TP.RowParallelLinear(act, self.Down.Data, self.s_down, self.s_down_b, residual=x, name="TpFfnDown")


class OaTpGptModel(OaModule):
    def __init__(self, cfg: OaGptConfig, mesh: OaDeviceMesh, micro_batch: int, full: Optional[OaGptModel] = None,
                 arena_bytes: Optional[int] = None):
        super().__init__()
        self.Cfg, self.Mesh, self.Batch = cfg, mesh, micro_batch
        W, r = mesh.world, mesh.rank
        rows = micro_batch * cfg.SeqLen
        D, V = cfg.DModel, cfg.Vocab
        assert V % (8 * W) == 0
        self.Rows, self.RowsLocal, self.VocabLocal = rows, rows // W, V // W
        per_layer = 8 * (rows * D * 2 + 4096)
        need = cfg.NLayers * per_layer + rows * D * 2 + rows * D * 2 + W * rows * 12 + (1 << 20)
        self.Arena = TP.OaTpArena(mesh, arena_bytes or need)
        std = cfg.InitStd or 0.02
        self.Embed = self.RegisterParameter("embed.weight", F.RandN([V, D], std=std))
        self.Blocks = []
        blocks = OaModule()
        for i in range(cfg.NLayers):
            b = OaTpBlock(cfg, self.Arena, rows, full.Blocks[i] if full is not None else None)
            blocks.RegisterModule(str(i), b)
            self.Blocks.append(b)
        self.RegisterModule("blocks", blocks)
        self.LnFinal = self.RegisterModule("ln_final", OaRmsNorm(D, cfg.Eps))
        self.Head = self.RegisterParameter("head.weight", F.RandN([V // W, D], std=std))
        self.s_head, self.s_head_b = TP.OaTpAgSite(self.Arena, rows, D), TP.OaTpRsSite(self.Arena, rows, D)
        self.Stats = TP.OaTpStats(self.Arena, rows)
        if full is not None:
            self.Embed.Data.Tensor().copy_(full.Embed.Weight.Tensor())
            self.LnFinal.Weight.Data.Tensor().copy_(full.LnFinal.Weight.Tensor())
            self.Head.Data.Tensor().copy_(full.Head.Weight.Tensor()[r * (V // W):(r + 1) * (V // W)])

    def ReplicatedParameters(self):
        out = [self.Embed, self.LnFinal.Weight]
        for b in self.Blocks:
            out += [b.LnAttn.Weight, b.LnFfn.Weight]
        return out

    def LogitsLocal(self, ids: OaMatrix) -> OaMatrix:
        """ids [B, S] (the same on every rank) -> this rank's vocabulary slice of the logits [B*S, V/W]."""
        r = self.Mesh.rank
        flat = ids.Tensor().reshape(-1)[r * self.RowsLocal:(r + 1) * self.RowsLocal].contiguous()
        x = F.Embedding(self.Embed.Data, OaMatrix(flat), None, 0)
        batch, seq = ids.Size(0), ids.Size(1)
        for b in self.Blocks:
            x = b.Forward(x, batch, seq)
        h = self.LnFinal.Forward(x)
        return TP.ColumnParallelLinear(h, self.Head.Data, self.s_head, self.s_head_b, "TpHead")

    def Loss(self, ids: OaMatrix, targets: OaMatrix) -> OaMatrix:
        return TP.VocabParallelCrossEntropy(self.LogitsLocal(ids), targets, self.Mesh, self.Stats)

    def SyncReplicatedGrads(self) -> None:
        """Sum over the group the gradients of replicated parameters (each rank saw 1/W of the rows)."""
        if self.Mesh.world == 1:
            return
        for p in self.ReplicatedParameters():
            g = p.Data.GradTensor()
            if g is not None:
                dist.all_reduce(g, group=self.Mesh.group)

    def FlopsPerToken(self) -> float:
        c = self.Cfg
        ffn = (3 if c.Ffn == "swiglu" else 2) * c.DModel * c.DFf
        per_layer = 2 * (4 * c.DModel * c.DModel + ffn) + 2 * 2 * c.SeqLen * c.DModel / 2
        return 3.0 * (c.NLayers * per_layer + 2 * c.DModel * c.Vocab)
