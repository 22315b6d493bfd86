"""Autoregressive decoding with a per-layer KV cache for the decoder-only Transformer models.

The reference regenerates by re-running the whole context window for every token (greedy window generation,
Tutorial/Cpp/Ml/Nlp/TutorialNlpCommon.h:145-177; no KV cache anywhere in Source/).  Here the prompt is processed once with
the tiled attention kernel while its rotated keys and values go into the cache, and every further token costs one GEMV-
shaped pass over the weights plus one read of the cache (csrc/kernels/decode.cu).  `Generate` returns exactly what the
full-window recomputation returns (the tests compare the two).
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from ..core import fn_matrix as F
from ..core.matrix import OaMatrix
from ..ml import autograd as AG
from ..ml import fn_fused as FF
from ..models.gpt import OaGptModel
from ..ops import kernels as K


class OaKvCache:
    """Keys and values of every layer: [layers][batch, heads, max_seq, head_dim] in the model's dtype."""

    def __init__(self, layers: int, batch: int, heads: int, max_seq: int, head_dim: int, dtype, device):
        self.K = [torch.zeros((batch, heads, max_seq, head_dim), dtype=dtype, device=device) for _ in range(layers)]
        self.V = [torch.zeros((batch, heads, max_seq, head_dim), dtype=dtype, device=device) for _ in range(layers)]
        self.Length, self.MaxSeq, self.Batch = 0, max_seq, batch

    def Bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self.K + self.V)

    def Reset(self) -> None:
        self.Length = 0


def _skinny_linear(x: OaMatrix, w: OaMatrix, residual: Optional[OaMatrix] = None) -> OaMatrix:
    """x [m, K] @ W[N, K]^T for a handful of rows: computed as (W @ x^T)^T so that the weight rows fill the 128-row MMA
    tile and the few tokens sit on the narrow N side, with split-K spreading the weight stream over all SMs."""
    tx, tw = x.Tensor(), w.Tensor()
    if not tx.is_cuda or tx.dtype != torch.bfloat16 or tx.shape[0] > 64 or tx.shape[0] % 8:
        return F.Linear(x, w, None, residual=residual)
    yt = K.gemm(tw, tx)                                    # [N, m]
    y = K.contiguous(yt.t())
    if residual is not None:
        y = K.binary("add", y, residual.Tensor(), out=y)
    return OaMatrix(y)


class _GraphedStep:
    """One decode step captured in a CUDA graph.  The position lives on the device (`pos`, int32 [1]): RoPE, the cache
    append and the attention length read it inside their kernels and the graph's last node adds one, so replaying needs no
    host-side parameter.  `ids` is the static input, the captured function's result the static output."""

    def __init__(self, device, batch: int):
        self.pos = torch.zeros(1, dtype=torch.int32, device=device)
        self.ids = torch.zeros((batch, 1), dtype=torch.int32, device=device)
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self.out = None

    def run(self, ids: torch.Tensor, fn):
        self.ids.copy_(ids.reshape(self.ids.shape))
        if self.graph is None:
            fn(self.ids)                              # eager once: lazily created buffers (workspaces) exist before the capture
            self.pos.sub_(1)
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, capture_error_mode="thread_local"):
                self.out = fn(self.ids)
            self.graph = g
        self.graph.replay()
        return self.out


class OaGptDecoder:
    def __init__(self, model: OaGptModel, batch: int, max_seq: int, use_graph: bool = True):
        self.Model, self.Cfg = model, model.Cfg
        c = self.Cfg
        w = model.Embed.Weight.Tensor()
        self.Cache = OaKvCache(c.NLayers, batch, c.NHeads, max_seq, c.DModel // c.NHeads, w.dtype, w.device)
        self._graphed = _GraphedStep(w.device, batch) if use_graph and w.is_cuda and w.dtype == torch.bfloat16 else None
        self._pos_dev: Optional[torch.Tensor] = None      # set while a graphed step records / replays

    # ---- one block on new tokens
    def _block(self, i: int, x: OaMatrix, batch: int, s_new: int) -> OaMatrix:
        b = self.Model.Blocks[i]
        a = b.Attention
        H, hd, D = a.NumHeads, a.HeadDim, a.DModel
        pos0, pd = self.Cache.Length, self._pos_dev
        if pd is not None:
            pos0 = 0                                  # the device-resident position carries the offset
        h = b.LnAttn.Forward(x)
        qw, kw, vw = a.QProj.Weight.Tensor(), a.KProj.Weight.Tensor(), a.VProj.Weight.Tensor()
        step = D * D * qw.element_size()
        adjacent = kw.data_ptr() == qw.data_ptr() + step and vw.data_ptr() == kw.data_ptr() + step
        if s_new == 1 and a.QProj.Bias is None and h.Tensor().is_cuda and adjacent:
            packed = qw
            base = packed.untyped_storage()
            wqkv = torch.empty(0, dtype=packed.dtype, device=packed.device).set_(base, packed.storage_offset(), (3 * D, D), (D, 1))
            qkv = _skinny_linear(h, OaMatrix(wqkv))            # q, k, v weights are row slices of one packed tensor
        else:
            qkv = a.ProjectQkv(h)
        t = qkv.Tensor()
        if s_new > 1:
            # prompt: tiled attention over the new tokens (rotates q and k in place), then cache the rotated k and v
            assert pos0 == 0, "prefill starts an empty cache"
            attn = F.FlashAttentionPacked(qkv, batch, s_new, H, hd, causal=True, rope_theta=a.RopeTheta)
            K.kv_append(t[:, D:2 * D], t[:, 2 * D:], self.Cache.K[i], self.Cache.V[i], batch, s_new, 0)
        else:
            if a.RopeTheta > 0:
                K.rope_(t[:, : 2 * D], 2 * H, hd, 1, pos_offset=pos0, theta=a.RopeTheta, pos_dev=pd)
            K.kv_append(t[:, D:2 * D], t[:, 2 * D:], self.Cache.K[i], self.Cache.V[i], batch, 1, pos0, pos_dev=pd)
            attn = OaMatrix(K.decode_attn(t[:, :D], self.Cache.K[i], self.Cache.V[i], pos0 + 1, pos_dev=pd))
        o = a.OutProj
        if s_new == 1 and o.Bias is None:
            x = _skinny_linear(attn, o.Weight.Data, residual=x)
        else:
            x = F.Linear(attn, o.Weight.Data, o.Bias.Data if o.Bias else None, residual=x)
        if b.Moe is not None:
            return b.Moe.Forward(x)
        if b.FfnKind == "gelu":
            hh = b.LnFfn.Forward(x)
            return FF.FfnGelu(hh, b.Ffn1.Weight.Data, b.Ffn1.Bias.Data if b.Ffn1.Bias else None, b.Ffn2.Weight.Data,
                              b.Ffn2.Bias.Data if b.Ffn2.Bias else None, residual=x)
        if s_new == 1:
            f = b.Ffn
            hh = f.Norm.Forward(x)
            gate, up = _skinny_linear(hh, f.Gate.Weight.Data), _skinny_linear(hh, f.Up.Weight.Data)
            return _skinny_linear(F.SiluMul(gate, up), f.Down.Weight.Data, residual=x)
        return b.Ffn.Forward(x)

    def _forward(self, ids: torch.Tensor) -> torch.Tensor:
        """ids [B, s_new] int32 -> logits of the last new position [B, vocab]; the cache grows by s_new."""
        m = self.Model
        batch, s_new = ids.shape
        if self.Cache.Length + s_new > self.Cache.MaxSeq:
            raise ValueError("KV cache is full")
        with AG.OaGradNo():
            if m.PosEmbed is not None:
                pos = m.PosEmbed.Weight.Tensor()[self.Cache.Length:self.Cache.Length + s_new]
                x = F.Embedding(m.Embed.Weight.Data, OaMatrix(ids.contiguous()), OaMatrix(pos.contiguous()), s_new)
            else:
                x = F.Embedding(m.Embed.Weight.Data, OaMatrix(ids.contiguous()), None, s_new)
            for i in range(len(m.Blocks)):
                x = self._block(i, x, batch, s_new)
            self.Cache.Length += s_new
            last = x.Tensor().reshape(batch, s_new, -1)[:, -1].contiguous() if s_new > 1 else x.Tensor()
            return m.Head.Forward(m.LnFinal.Forward(OaMatrix(last))).Tensor()

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
            out = self._forward(ids)
            self.Cache.Length = length                  # the host-side length advances once per Step, not per recording
            self._graphed.pos.add_(1)
            return out
        finally:
            self._pos_dev = None

    def Step(self, ids: torch.Tensor) -> torch.Tensor:
        """One token per sequence.  On CUDA (bf16, learned-position-free models) the step replays a captured graph; the
        returned logits tensor is then the graph's static output and is overwritten by the next Step."""
        g = self._graphed
        if g is None or self.Model.PosEmbed is not None or ids.numel() != g.ids.numel():
            return self._forward(ids.reshape(-1, 1))
        if self.Cache.Length + 1 > self.Cache.MaxSeq:
            raise ValueError("KV cache is full")
        out = g.run(ids, self._graph_body)
        self.Cache.Length += 1
        return out

    def Generate(self, prompt: torch.Tensor, new_tokens: int) -> torch.Tensor:
        """Greedy decoding: prompt [B, S] int32 -> [B, S + new_tokens]."""
        out = [prompt]
        logits = self.Prefill(prompt)
        for _ in range(new_tokens):
            nxt = logits.float().argmax(-1).to(torch.int32).reshape(-1, 1)
            out.append(nxt)
            if len(out) - 1 < new_tokens:
                logits = self.Step(nxt)
        return torch.cat(out, 1)
