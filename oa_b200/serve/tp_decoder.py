"""Tensor-parallel autoregressive decoding: replicated activations, sharded weights and KV cache, one-shot all-reduce.

Every rank holds the attention heads [r*H/W, (r+1)*H/W), the FFN columns and the vocabulary rows of an OaTpGptModel
(parallel/tp_model.py) plus the KV cache of its own heads.  A decode step keeps the [batch, d_model] activations replicated:
the column-parallel projections need no communication, the row-parallel ones produce partial sums that one kernel per
projection all-reduces through peer memory (csrc/kernels/comm.cu, peer_allreduce_oneshot_kernel: push to every rank's
staging slot, per-CTA counters, fp32 sum + residual) - two such kernels per layer.  The prompt is processed with the same
sharding, its large partial sums go through NCCL.  Greedy sampling takes the arg-max over the gathered vocabulary shards.
"""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.distributed as dist

from .. import _native as N
from ..core import fn_matrix as F
from ..core.matrix import OaMatrix
from ..ml import autograd as AG
from ..ops import kernels as K
from ..parallel.mesh import OaDeviceMesh
from ..parallel.tp_model import OaTpGptModel
from .decoder import OaKvCache, _GraphedStep, _skinny_linear


class OaOneShotAllReduce:
    """out = sum over ranks of a small bf16 tensor (+ residual) in ONE kernel; call order must be the same on every rank."""
    MAX_CTAS = 64

    def __init__(self, mesh: OaDeviceMesh, max_elems: int):
        self.Mesh = mesh
        self.SlotElems = (int(max_elems) + 7) // 8 * 8
        if self.SlotElems > self.MAX_CTAS * 2048:
            raise ValueError("one-shot all-reduce is for messages of at most 131072 elements")
        self._slots = mesh.AllocSymmetric(2 * mesh.world * self.SlotElems * 2)
        self._counters = mesh.AllocSymmetric(self.MAX_CTAS * 8)
        self._counters.view(torch.int64, self.MAX_CTAS).zero_()
        self._sync = torch.zeros(2 + self.MAX_CTAS, dtype=torch.int64, device=mesh.device)
        torch.cuda.synchronize()
        if mesh.world > 1:
            dist.barrier(group=mesh.group)

    def __call__(self, src: torch.Tensor, residual: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        m = self.Mesh
        assert src.dtype == torch.bfloat16 and src.is_contiguous() and src.numel() % 8 == 0 and src.numel() <= self.SlotElems
        out = torch.empty_like(src) if out is None else out
        K._launch(N.require().oa_peer_allreduce_oneshot(self._slots.ptr_array, self._counters.ptr_array, src.data_ptr(), N.ptr(residual),
                                                        out.data_ptr(), self._sync.data_ptr(), src.numel(), self.SlotElems, m.world, m.rank,
                                                        self.MAX_CTAS, K.status_word(m.device).data_ptr(), N.stream()),
                  "oa_peer_allreduce_oneshot")
        return out


class OaTpGptDecoder:
    def __init__(self, model: OaTpGptModel, batch: int, max_seq: int, use_graph: bool = True):
        self.Model, self.Cfg, self.Mesh = model, model.Cfg, model.Mesh
        c, W = self.Cfg, model.Mesh.world
        self.HeadsLocal, self.HeadDim = c.NHeads // W, c.DModel // c.NHeads
        w = model.Embed.Data.Tensor()
        self.Cache = OaKvCache(c.NLayers, batch, self.HeadsLocal, max_seq, self.HeadDim, w.dtype, w.device)
        self.AllReduce = OaOneShotAllReduce(model.Mesh, batch * c.DModel) if W > 1 and batch * c.DModel <= 131072 else None
        # the decode step replays as a CUDA graph when its all-reduces are the graph-safe one-shot kernels
        self._graphed = _GraphedStep(w.device, batch) if use_graph and w.is_cuda and (W == 1 or self.AllReduce is not None) else None
        self._pos_dev: Optional[torch.Tensor] = None

    def _reduce(self, partial: torch.Tensor, residual: torch.Tensor, small: bool) -> OaMatrix:
        if self.Mesh.world == 1:
            return OaMatrix(K.binary("add", partial, residual))
        if small and self.AllReduce is not None:
            return OaMatrix(self.AllReduce(partial, residual))
        dist.all_reduce(partial, group=self.Mesh.group)
        return OaMatrix(K.binary("add", partial, residual, out=partial))

    def _block(self, i: int, x: OaMatrix, batch: int, s_new: int) -> OaMatrix:
        b = self.Model.Blocks[i]
        Hl, hd = self.HeadsLocal, self.HeadDim
        Dl = Hl * hd
        pos0, pd = self.Cache.Length, self._pos_dev
        if pd is not None:
            pos0 = 0
        small = s_new == 1
        lin = _skinny_linear if small else (lambda a, w_: F.Linear(a, w_, None))
        h = b.LnAttn.Forward(x)
        qkv = lin(h, b.Qkv.Data)                                   # [rows, 3 * Dl]: this rank's heads, q | k | v
        t = qkv.Tensor()
        if s_new > 1:
            assert pos0 == 0, "prefill starts an empty cache"
            attn = F.FlashAttentionPacked(qkv, batch, s_new, Hl, hd, causal=True, rope_theta=self.Cfg.RopeTheta)
            K.kv_append(t[:, Dl:2 * Dl], t[:, 2 * Dl:], self.Cache.K[i], self.Cache.V[i], batch, s_new, 0)
        else:
            K.rope_(t[:, : 2 * Dl], 2 * Hl, hd, 1, pos_offset=pos0, theta=self.Cfg.RopeTheta, pos_dev=pd)
            K.kv_append(t[:, Dl:2 * Dl], t[:, 2 * Dl:], self.Cache.K[i], self.Cache.V[i], batch, 1, pos0, pos_dev=pd)
            attn = OaMatrix(K.decode_attn(t[:, :Dl], self.Cache.K[i], self.Cache.V[i], pos0 + 1, pos_dev=pd))
        x = self._reduce(F._c(lin(attn, b.Out.Data).Tensor()), x.Tensor(), small)
        h = b.LnFfn.Forward(x)
        up = lin(h, b.Up.Data)
        act = F.Swiglu(up) if b.Gated else F.Gelu(up)
        return self._reduce(F._c(lin(act, b.Down.Data).Tensor()), x.Tensor(), small)

    def _forward(self, ids: torch.Tensor) -> torch.Tensor:
        """ids [B, s_new] int32 (the same on every rank) -> logits of the last new position [B, vocab] (gathered)."""
        return self._gather(self._forward_local(ids), ids.shape[0])

    def _gather(self, local: torch.Tensor, batch: int) -> torch.Tensor:
        W = self.Mesh.world
        if W == 1:
            return local
        parts = torch.empty((W,) + tuple(local.shape), dtype=local.dtype, device=local.device)
        dist.all_gather_into_tensor(parts, local, group=self.Mesh.group)
        return parts.permute(1, 0, 2).reshape(batch, -1)

    def _forward_local(self, ids: torch.Tensor) -> torch.Tensor:
        """This rank's vocabulary shard of the logits [B, vocab / W]."""
        m = self.Model
        batch, s_new = ids.shape
        if self.Cache.Length + s_new > self.Cache.MaxSeq:
            raise ValueError("KV cache is full")
        with AG.OaGradNo():
            x = F.Embedding(m.Embed.Data, OaMatrix(ids.contiguous().reshape(-1)), None, 0)
            for i in range(len(m.Blocks)):
                x = self._block(i, x, batch, s_new)
            self.Cache.Length += s_new
            last = x.Tensor().reshape(batch, s_new, -1)[:, -1].contiguous() if s_new > 1 else x.Tensor()
            h = m.LnFinal.Forward(OaMatrix(last))
            return (_skinny_linear(h, m.Head.Data) if s_new == 1 else F.Linear(h, m.Head.Data, None)).Tensor().contiguous()

    def Prefill(self, prompt: torch.Tensor) -> torch.Tensor:
        self.Cache.Reset()
        out = self._forward(prompt)
        if self._graphed is not None:
            self._graphed.pos.fill_(self.Cache.Length)
        return out

    def _graph_body(self, ids: torch.Tensor) -> torch.Tensor:
        self._pos_dev = self._graphed.pos
        try:
            length = self.Cache.Length
            out = self._forward_local(ids)
            self.Cache.Length = length
            self._graphed.pos.add_(1)
            return out
        finally:
            self._pos_dev = None

    def Step(self, ids: torch.Tensor) -> torch.Tensor:
        g = self._graphed
        if g is None or ids.numel() != g.ids.numel():
            return self._forward(ids.reshape(-1, 1))
        if self.Cache.Length + 1 > self.Cache.MaxSeq:
            raise ValueError("KV cache is full")
        local = g.run(ids, self._graph_body)            # the captured step ends at the local logits; the gather runs eagerly
        self.Cache.Length += 1
        return self._gather(local, g.ids.shape[0])

    def Generate(self, prompt: torch.Tensor, new_tokens: int) -> torch.Tensor:
        """Greedy decoding: prompt [B, S] int32 -> [B, S + new_tokens] (identical on every rank)."""
        out = [prompt]
        logits = self.Prefill(prompt)
        for _ in range(new_tokens):
            nxt = logits.float().argmax(-1).to(torch.int32).reshape(-1, 1)
            out.append(nxt)
            if len(out) - 1 < new_tokens:
                logits = self.Step(nxt)
        return torch.cat(out, 1)
