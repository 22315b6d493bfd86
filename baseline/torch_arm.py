"""The library baseline of the benchmark: the same five model configurations written in plain PyTorch.

Nothing in this file touches the repo's kernels or engine.  Matrix products go to cuBLAS through `F.linear`, attention to
`F.scaled_dot_product_attention` (cuDNN / flash back end), normalisation and losses to torch's own kernels, the optimizer
is `torch.optim.AdamW(fused=True)` over fp32 master copies of bf16 parameters, data parallelism is
`DistributedDataParallel` over NCCL, tensor parallelism is NCCL all-gather / reduce-scatter around column / row
parallel linears with sequence-sharded norms and a vocabulary-parallel cross-entropy, and expert parallelism is
`all_to_all_single` around a grouped expert product.  `bench.py --impl torch` runs it under the same timing protocol as
the default arm, and the default arm runs it first to fill `vs_baseline`.
"""
from __future__ import annotations

import math
import os
from dataclasses import dataclass
from typing import Optional

import torch
import torch.distributed as dist
import torch.nn as nn
import torch.nn.functional as F


@dataclass
class TorchLmConfig:
    vocab: int
    d_model: int
    n_layers: int
    n_heads: int
    d_ff: int
    seq_len: int
    norm: str = "rms"            # "rms" | "layer"
    ffn: str = "gelu"            # "gelu" | "swiglu"
    rope_theta: float = 10000.0  # 0: learned positions
    bias: bool = False
    eps: float = 1e-5
    n_experts: int = 0
    top_k: int = 2
    expert_ff: int = 0
    shared_experts: int = 0
    aux_alpha: float = 0.0


def config_by_number(k: int) -> TorchLmConfig:
    if k == 1:
        return TorchLmConfig(256, 128, 4, 4, 512, 128, "layer", "gelu", 0.0, True)
    if k == 2:
        return TorchLmConfig(32000, 1024, 24, 16, 4096, 2048)
    if k == 3:
        return TorchLmConfig(32000, 2048, 16, 16, 1408, 2048, "rms", "swiglu", n_experts=64, top_k=2, expert_ff=1408,
                             shared_experts=1, aux_alpha=0.01)
    if k == 5:
        return TorchLmConfig(32000, 4096, 32, 32, 11008, 4096, "rms", "swiglu")
    raise ValueError(k)


def _norm(kind: str, d: int, eps: float) -> nn.Module:
    return nn.LayerNorm(d, eps=eps) if kind == "layer" else nn.RMSNorm(d, eps=eps)


def _rope_tables(seq: int, hd: int, theta: float, device, dtype):
    inv = theta ** (-torch.arange(0, hd // 2, device=device, dtype=torch.float32) * 2.0 / hd)
    ang = torch.arange(seq, device=device, dtype=torch.float32)[:, None] * inv[None]
    return torch.cos(ang).to(dtype), torch.sin(ang).to(dtype)


def _apply_rope(x, cos, sin):
    """x [B, H, S, hd]; rotate-half pairs (i, i + hd/2)."""
    h = x.shape[-1] // 2
    x1, x2 = x[..., :h], x[..., h:]
    return torch.cat((x1 * cos - x2 * sin, x2 * cos + x1 * sin), -1)


# ------------------------------------------------------------------------------------------------ tensor-parallel pieces
class _GatherSeq(torch.autograd.Function):
    """All-gather of sequence-sharded rows in forward, reduce-scatter of the gradient in backward."""

    @staticmethod
    def forward(ctx, x):
        w = dist.get_world_size()
        out = x.new_empty((x.shape[0] * w, *x.shape[1:]))
        dist.all_gather_into_tensor(out, x.contiguous())
        return out

    @staticmethod
    def backward(ctx, g):
        w = dist.get_world_size()
        out = g.new_empty((g.shape[0] // w, *g.shape[1:]))
        dist.reduce_scatter_tensor(out, g.contiguous())
        return out


class _ScatterSeq(torch.autograd.Function):
    """Reduce-scatter of partial sums onto sequence shards in forward, all-gather of the gradient in backward."""

    @staticmethod
    def forward(ctx, x):
        w = dist.get_world_size()
        out = x.new_empty((x.shape[0] // w, *x.shape[1:]))
        dist.reduce_scatter_tensor(out, x.contiguous())
        return out

    @staticmethod
    def backward(ctx, g):
        w = dist.get_world_size()
        out = g.new_empty((g.shape[0] * w, *g.shape[1:]))
        dist.all_gather_into_tensor(out, g.contiguous())
        return out


class _VocabParallelCe(torch.autograd.Function):
    """Mean cross-entropy over logits whose vocabulary axis is sharded over the ranks."""

    @staticmethod
    def forward(ctx, logits, target, v0):
        lf = logits.float()
        mx = lf.max(-1).values
        dist.all_reduce(mx, op=dist.ReduceOp.MAX)
        ex = torch.exp(lf - mx[:, None])
        den = ex.sum(-1)
        dist.all_reduce(den)
        local = target - v0
        ok = (local >= 0) & (local < logits.shape[1])
        picked = torch.where(ok, lf.gather(1, local.clamp(0, logits.shape[1] - 1)[:, None]).squeeze(1), torch.zeros_like(mx))
        dist.all_reduce(picked)
        loss = (torch.log(den) + mx - picked).mean()
        ctx.save_for_backward(ex, den, local, ok)
        ctx.dtype = logits.dtype
        return loss

    @staticmethod
    def backward(ctx, g):
        ex, den, local, ok = ctx.saved_tensors
        p = ex / den[:, None]
        rows = torch.nonzero(ok).squeeze(1)
        p[rows, local[rows]] -= 1.0
        return (p * (g / p.shape[0])).to(ctx.dtype), None, None


# ------------------------------------------------------------------------------------------------ blocks
class Attention(nn.Module):
    def __init__(self, c: TorchLmConfig, tp: int):
        super().__init__()
        self.c, self.tp = c, tp
        self.heads = c.n_heads // tp
        self.hd = c.d_model // c.n_heads
        self.qkv = nn.Linear(c.d_model, 3 * c.d_model // tp, bias=c.bias)
        self.out = nn.Linear(c.d_model // tp, c.d_model, bias=c.bias and tp == 1)

    def forward(self, x, batch, seq, rope):
        q, k, v = self.qkv(x).view(batch, seq, 3, self.heads, self.hd).permute(2, 0, 3, 1, 4)
        if rope is not None:
            q, k = _apply_rope(q, *rope), _apply_rope(k, *rope)
        o = F.scaled_dot_product_attention(q, k, v, is_causal=True)
        return self.out(o.transpose(1, 2).reshape(batch * seq, self.heads * self.hd))


class Mlp(nn.Module):
    def __init__(self, c: TorchLmConfig, d_ff: int, tp: int):
        super().__init__()
        self.swiglu = c.ffn == "swiglu"
        self.up = nn.Linear(c.d_model, (2 if self.swiglu else 1) * d_ff // tp, bias=c.bias)
        self.down = nn.Linear(d_ff // tp, c.d_model, bias=c.bias and tp == 1)

    def forward(self, x):
        h = self.up(x)
        if self.swiglu:
            g, u = h.chunk(2, -1)
            h = F.silu(g) * u
        else:
            h = F.gelu(h, approximate="tanh")
        return self.down(h)


def _grouped_linear(x, w, counts):
    """x [T, in] sorted by expert, w [E, out, in], counts: python list of rows per expert."""
    if hasattr(torch, "_grouped_mm") and x.dtype == torch.bfloat16:
        try:
            offs = torch.tensor(counts, device=x.device, dtype=torch.int32).cumsum(0).to(torch.int32)
            return torch._grouped_mm(x, w.transpose(1, 2), offs=offs)
        except Exception:
            pass
    outs, r = [], 0
    for e, n in enumerate(counts):
        outs.append(F.linear(x[r:r + n], w[e]))
        r += n
    return torch.cat(outs, 0)


class MoE(nn.Module):
    """Dropless top-k softmax-router MoE with SwiGLU experts, optional shared experts and a load-balance loss.  With
    `ep` > 1 the experts are sharded over the ranks and rows travel through two `all_to_all_single` calls each way."""

    def __init__(self, c: TorchLmConfig, ep: int):
        super().__init__()
        self.c, self.ep = c, ep
        self.e_local = c.n_experts // ep
        self.router = nn.Linear(c.d_model, c.n_experts, bias=False)
        self.w_gate_up = nn.Parameter(torch.empty(self.e_local, 2 * c.expert_ff, c.d_model))
        self.w_down = nn.Parameter(torch.empty(self.e_local, c.d_model, c.expert_ff))
        self.shared = Mlp(c, c.expert_ff * c.shared_experts, 1) if c.shared_experts else None
        self.aux = None

    def _experts(self, rows, counts):
        h = _grouped_linear(rows, self.w_gate_up, counts)
        g, u = h.chunk(2, -1)
        return _grouped_linear(F.silu(g) * u, self.w_down, counts)

    def forward(self, x):
        c = self.c
        T = x.shape[0]
        probs = F.softmax(self.router(x).float(), -1)
        top_p, top_e = probs.topk(c.top_k, -1)
        wts = (top_p / top_p.sum(-1, keepdim=True)).to(x.dtype)
        flat_e = top_e.reshape(-1)
        order = torch.argsort(flat_e, stable=True)
        counts_t = torch.bincount(flat_e, minlength=c.n_experts)
        if c.aux_alpha > 0:
            frac = counts_t.float() / (T * c.top_k)
            self.aux = c.aux_alpha * c.n_experts * (frac * probs.mean(0)).sum()
        rows = x[order // c.top_k]
        if self.ep == 1:
            out_rows = self._experts(rows, counts_t.tolist())
        else:
            w = self.ep
            recv_counts_t = torch.empty_like(counts_t)
            dist.all_to_all_single(recv_counts_t, counts_t)
            send = counts_t.view(w, self.e_local).sum(1).tolist()
            rc = recv_counts_t.view(w, self.e_local)
            recv = rc.sum(1).tolist()
            got = _AllToAll.apply(rows, send, recv)
            # rows arrive rank-major; regroup expert-major for the grouped product
            src_e = torch.repeat_interleave(torch.arange(self.e_local, device=x.device).repeat(w), rc.reshape(-1))
            perm = torch.argsort(src_e, stable=True)
            y = self._experts(got[perm], rc.sum(0).tolist())
            back = torch.empty_like(y)
            back[perm] = y
            out_rows = _AllToAll.apply(back, recv, send)
        contrib = out_rows * wts.reshape(-1)[order][:, None]
        out = torch.zeros_like(x).index_add_(0, order // c.top_k, contrib)
        if self.shared is not None:
            out = out + self.shared(x)
        return out


class _AllToAll(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, send, recv):
        ctx.send, ctx.recv = send, recv
        out = x.new_empty((sum(recv), x.shape[1]))
        dist.all_to_all_single(out, x.contiguous(), output_split_sizes=recv, input_split_sizes=send)
        return out

    @staticmethod
    def backward(ctx, g):
        out = g.new_empty((sum(ctx.send), g.shape[1]))
        dist.all_to_all_single(out, g.contiguous(), output_split_sizes=ctx.send, input_split_sizes=ctx.recv)
        return out, None, None


class Block(nn.Module):
    def __init__(self, c: TorchLmConfig, tp: int, ep: int):
        super().__init__()
        self.tp = tp
        self.n1, self.n2 = _norm(c.norm, c.d_model, c.eps), _norm(c.norm, c.d_model, c.eps)
        self.attn = Attention(c, tp)
        self.moe = MoE(c, ep) if c.n_experts else None
        self.mlp = None if c.n_experts else Mlp(c, c.d_ff, tp)

    def forward(self, x, batch, seq, rope):
        if self.tp == 1:
            x = x + self.attn(self.n1(x), batch, seq, rope)
            return x + (self.moe(self.n2(x)) if self.moe is not None else self.mlp(self.n2(x)))
        x = x + _ScatterSeq.apply(self.attn(_GatherSeq.apply(self.n1(x)), batch, seq, rope))
        return x + _ScatterSeq.apply(self.mlp(_GatherSeq.apply(self.n2(x))))


class TorchLm(nn.Module):
    def __init__(self, c: TorchLmConfig, tp: int = 1, ep: int = 1):
        super().__init__()
        self.c, self.tp, self.ep = c, tp, ep
        self.embed = nn.Embedding(c.vocab, c.d_model)
        self.pos = nn.Embedding(c.seq_len, c.d_model) if c.rope_theta <= 0 else None
        self.blocks = nn.ModuleList([Block(c, tp, ep) for _ in range(c.n_layers)])
        self.norm = _norm(c.norm, c.d_model, c.eps)
        self.head = nn.Linear(c.d_model, c.vocab // tp, bias=c.bias and tp == 1)
        for p in self.parameters():
            if p.dim() >= 2:
                nn.init.normal_(p, 0.0, 0.02)
        self._rope = None

    def loss(self, ids, tgt):
        c = self.c
        batch, seq = ids.shape
        x = self.embed(ids).view(batch * seq, c.d_model)
        if self.pos is not None:
            x = x + self.pos.weight[:seq].repeat(batch, 1)
        rope = None
        if c.rope_theta > 0:
            if self._rope is None or self._rope[0].shape[0] != seq or self._rope[0].dtype != x.dtype:
                self._rope = _rope_tables(seq, c.d_model // c.n_heads, c.rope_theta, x.device, x.dtype)
            rope = self._rope
        if self.tp > 1:                      # sequence-sharded residual stream (batch 1: rows = positions)
            r = dist.get_rank()
            n = batch * seq // self.tp
            x = x[r * n:(r + 1) * n]
        for b in self.blocks:
            x = b(x, batch, seq, rope)
        x = self.norm(x)
        if self.tp > 1:
            logits = self.head(_GatherSeq.apply(x))
            return _VocabParallelCe.apply(logits, tgt.reshape(-1).long(), dist.get_rank() * (c.vocab // self.tp))
        loss = F.cross_entropy(self.head(x), tgt.reshape(-1).long())
        if c.n_experts and c.aux_alpha > 0:
            for b in self.blocks:
                loss = loss + b.moe.aux
        return loss

    forward = loss

    def replicated_parameters(self):
        """Parameters that every tensor-parallel rank holds whole (their gradients need a sum over the ranks)."""
        out = [self.embed.weight] + list(self.norm.parameters())
        for b in self.blocks:
            out += list(b.n1.parameters()) + list(b.n2.parameters())
        return out

    def expert_parameters(self):
        return [p for b in self.blocks if b.moe is not None for p in (b.moe.w_gate_up, b.moe.w_down)]


# ------------------------------------------------------------------------------------------------ Mamba-3 (config 4)
@dataclass
class TorchMamba3Config:
    vocab: int = 32000
    d_model: int = 1536
    n_layers: int = 32
    d_state: int = 128
    expand: int = 2
    headdim: int = 64
    seq_len: int = 4096
    chunk: int = 128
    eps: float = 1e-5
    conv_width: int = 4
    a_log: bool = True


def _softplus_inv(y):
    return y + torch.log(-torch.expm1(-y))


class Mamba3Mixer(nn.Module):
    """The reference's Mamba-3 SISO mixer (data-dependent decay, trapezoid update, rotary state phase, per-head skip and
    gated RMSNorm) in its chunked state-space-duality form, written with tensor expressions and batched matmuls; autograd
    differentiates it.  Recurrence: Source/Private/Oa/Ml/Shader/Compute/Nn/Ssm/Mamba3/Mamba3SisoFwd.slang:9-18."""

    def __init__(self, c: TorchMamba3Config):
        super().__init__()
        self.c = c
        self.d_inner = c.expand * c.d_model
        self.heads = self.d_inner // c.headdim
        self.angles = (int(c.d_state * 0.5) & ~1) // 2
        self.d_in_proj = 2 * self.d_inner + 2 * c.d_state + 3 * self.heads + self.angles
        self.in_proj = nn.Linear(c.d_model, self.d_in_proj, bias=False)
        self.out_proj = nn.Linear(self.d_inner, c.d_model, bias=False)
        u = torch.rand(self.heads) * (math.log(1e-1) - math.log(1e-3)) + math.log(1e-3)
        self.dt_bias = nn.Parameter(_softplus_inv(torch.exp(u)))
        self.B_bias = nn.Parameter(torch.ones(self.heads, c.d_state))
        self.C_bias = nn.Parameter(torch.ones(self.heads, c.d_state))
        self.D = nn.Parameter(torch.ones(self.heads))
        self.norm_weight = nn.Parameter(torch.ones(self.d_inner))
        cw = self.d_inner + 2 * c.d_state
        self.conv = nn.Conv1d(cw, cw, c.conv_width, groups=cw, padding=c.conv_width - 1, bias=False) if c.conv_width else None
        self.A_log = nn.Parameter(torch.log(1.0 + 15.0 * torch.rand(self.heads))) if c.a_log else None

    def forward(self, u, batch, seq):
        c, H, P, N, A, Q = self.c, self.heads, self.c.headdim, self.c.d_state, self.angles, self.c.chunk
        proj = self.in_proj(u).view(batch, seq, self.d_in_proj)
        z, x, Bn, Cn, dd_dt, dd_a, trap, ang = proj.split([self.d_inner, self.d_inner, N, N, H, H, H, A], -1)
        if self.conv is not None:
            xbc = torch.cat((x, Bn, Cn), -1).transpose(1, 2)
            xbc = F.silu(self.conv(xbc)[..., :seq]).transpose(1, 2)
            x, Bn, Cn = xbc.split([self.d_inner, N, N], -1)
        f32 = torch.float32
        dt = F.softplus(dd_dt.to(f32) + self.dt_bias.to(f32)).clamp(1e-3, 0.1)
        if self.A_log is not None:
            adt = -torch.exp(self.A_log.to(f32)) * dt
        else:
            da = dd_a.to(f32)
            heavy = torch.where(da >= 0, 1.0 + da, 1.0 / (1.0 - da.clamp(max=0.0)))
            adt = torch.minimum(-heavy, torch.full_like(heavy, -1e-4)) * dt
        Bn = F.rms_norm(Bn.to(f32), (N,), eps=c.eps)
        Cn = F.rms_norm(Cn.to(f32), (N,), eps=c.eps)
        tr = torch.sigmoid(trap.to(f32))
        gamma, late = dt * tr, dt * (1.0 - tr)
        scale = gamma + torch.cat((late[:, 1:], torch.zeros_like(late[:, :1])), 1)
        theta = torch.cumsum(ang.to(f32)[:, :, None, :] * dt[..., None], 1)
        cos, sin = torch.cos(theta), torch.sin(theta)

        def rot(v):
            h = v[..., :2 * A].reshape(*v.shape[:-1], A, 2)
            r = torch.stack((h[..., 0] * cos - h[..., 1] * sin, h[..., 0] * sin + h[..., 1] * cos), -1).reshape(*v.shape[:-1], 2 * A)
            return torch.cat((r, v[..., 2 * A:]), -1)

        Ct = rot(Cn[:, :, None, :] + self.C_bias.to(f32))          # [B, L, H, N]
        Bt = rot(Bn[:, :, None, :] + self.B_bias.to(f32))
        nC = seq // Q
        ch = lambda t: t.reshape(batch, nC, Q, H, *t.shape[3:]).transpose(2, 3)      # [B, nC, H, Q, ...]
        xh = x.reshape(batch, seq, H, P)
        cum = torch.cumsum(ch(adt), -1)                             # [B, nC, H, Q]
        Cc, Bc, Xc = ch(Ct).to(u.dtype), ch(Bt).to(u.dtype), ch(xh)
        G = torch.matmul(Cc, Bc.transpose(-1, -2)).float()           # [B, nC, H, Q, Q]
        tri = torch.tril(torch.ones(Q, Q, device=u.device, dtype=torch.bool), -1)
        E = torch.exp((cum[..., :, None] - cum[..., None, :]).masked_fill(~tri, float("-inf")))
        M = G * E * ch(scale)[..., None, :]
        diag = self.D.to(f32)[None, None, :, None] + ch(gamma) * (ch(Ct) * ch(Bt)).sum(-1)
        M = M + torch.diag_embed(diag)
        Y = torch.matmul(M.to(u.dtype), Xc).float()                  # [B, nC, H, Q, P]
        w = torch.exp(cum[..., -1:] - cum) * ch(scale)
        S = torch.matmul((Xc.float() * w[..., None]).to(u.dtype).transpose(-1, -2), Bc).float()   # [B, nC, H, P, N]
        dec = torch.exp(cum[..., -1])                               # [B, nC, H]
        hin, state = [], torch.zeros(batch, H, P, N, device=u.device, dtype=f32)
        for k in range(nC):
            hin.append(state)
            state = state * dec[:, k, :, None, None] + S[:, k]
        Hin = torch.stack(hin, 1)                                   # [B, nC, H, P, N]
        Y = Y + torch.matmul((ch(Ct) * torch.exp(cum)[..., None]).to(u.dtype), Hin.to(u.dtype).transpose(-1, -2)).float()
        y = Y.transpose(2, 3).reshape(batch, seq, H, P)
        y = y * F.silu(z.view(batch, seq, H, P).float())
        y = F.rms_norm(y.reshape(batch, seq, self.d_inner), (self.d_inner,), self.norm_weight.float(), c.eps)
        return self.out_proj(y.to(u.dtype).view(batch * seq, self.d_inner))


class TorchMamba3Lm(nn.Module):
    def __init__(self, c: TorchMamba3Config):
        super().__init__()
        self.c = c
        self.embed = nn.Embedding(c.vocab, c.d_model)
        self.norms = nn.ModuleList([nn.RMSNorm(c.d_model, eps=c.eps) for _ in range(c.n_layers)])
        self.mixers = nn.ModuleList([Mamba3Mixer(c) for _ in range(c.n_layers)])
        self.norm = nn.RMSNorm(c.d_model, eps=c.eps)
        self.head = nn.Linear(c.d_model, c.vocab, bias=False)
        for p in self.parameters():
            if p.dim() >= 2 and p.shape[0] > 64:
                nn.init.normal_(p, 0.0, 0.02)

    def loss(self, ids, tgt):
        from torch.utils.checkpoint import checkpoint
        batch, seq = ids.shape
        x = self.embed(ids).view(batch * seq, self.c.d_model)
        for n, m in zip(self.norms, self.mixers):
            x = x + checkpoint(lambda t, n=n, m=m: m(n(t), batch, seq), x, use_reentrant=False)
        return F.cross_entropy(self.head(self.norm(x)), tgt.reshape(-1).long())

    forward = loss


# ------------------------------------------------------------------------------------------------ training step
class TorchTrainer:
    """bf16 parameters with fp32 master copies and fused AdamW; DDP / TP / EP as the configuration asks; the whole step
    is captured as a CUDA graph on one GPU when capture succeeds."""

    def __init__(self, config: int, world: int, device, micro_batch: int, accum: int = 1, fp32: bool = False,
                 layers: int = 0, seq: int = 0, graph: bool = True):
        self.config, self.world, self.dev, self.accum = config, world, device, accum
        dtype = torch.float32 if fp32 else torch.bfloat16
        torch.manual_seed(20260714)
        tp = world if config == 5 else 1
        ep = world if config == 3 else 1
        with torch.device(device):
            if config == 4:
                c = TorchMamba3Config()
                if layers:
                    c.n_layers = layers
                if seq:
                    c.seq_len = seq
                self.model = TorchMamba3Lm(c)
            else:
                c = config_by_number(config)
                if layers:
                    c.n_layers = layers
                if seq:
                    c.seq_len = seq
                self.model = TorchLm(c, tp, ep)
        self.cfg = c
        self.model.to(dtype)
        self.fp32 = fp32
        self.params = [p for p in self.model.parameters()]
        self.masters = self.params if fp32 else [p.detach().float().clone() for p in self.params]
        # The two largest models on ONE GPU (64 experts resident, or all of the 7B model) leave no room for a second fp32
        # copy of every gradient: there the update walks the parameters one at a time, each with its own fused AdamW.
        self.low_mem = (not fp32) and world == 1 and config in (3, 5) and not layers
        if not fp32 and not self.low_mem:
            for m in self.masters:
                m.grad = torch.zeros_like(m)
        self.run = self.model
        self.sync_lists = []
        if world > 1 and config in (2, 4, 1):
            from torch.nn.parallel import DistributedDataParallel as DDP
            self.ddp = DDP(self.model, device_ids=[device.index], gradient_as_bucket_view=True, bucket_cap_mb=64)
            self.run = self.ddp
        elif world > 1 and config == 5:
            self.sync_lists = [(self.model.replicated_parameters(), 1.0)]
        elif world > 1 and config == 3:
            ex = {id(p) for p in self.model.expert_parameters()}
            self.sync_lists = [([p for p in self.params if id(p) not in ex], 1.0 / world)]
            self.expert_scale = 1.0 / world
        self.use_graph = graph and world == 1 and config != 3 and not self.low_mem
        wd = 0.0 if config == 1 else 0.1
        if self.low_mem:
            self.opts = [torch.optim.AdamW([m], lr=3e-4, weight_decay=wd, fused=True) for m in self.masters]
        else:
            self.opt = torch.optim.AdamW(self.masters, lr=3e-4, weight_decay=wd, fused=True, capturable=self.use_graph)
        self.ids = torch.zeros((micro_batch, c.seq_len), dtype=torch.int32, device=device)
        self.tgt = torch.zeros((micro_batch, c.seq_len), dtype=torch.int32, device=device)
        self.loss = torch.zeros((), device=device)
        self.graph = None
        self.micro_feed = None

    def _fwd_bwd(self):
        loss = self.run(self.ids, self.tgt)          # through the DDP wrapper when there is one (its hooks reduce the gradients)
        (loss / self.accum if self.accum > 1 else loss).backward()
        return loss.detach()

    @torch.no_grad()
    def _optim(self):
        if self.sync_lists:
            for plist, scale in self.sync_lists:
                flat = torch.cat([p.grad.reshape(-1) for p in plist])
                dist.all_reduce(flat)
                if scale != 1.0:
                    flat *= scale
                off = 0
                for p in plist:
                    n = p.numel()
                    p.grad.copy_(flat[off:off + n].view_as(p))
                    off += n
            if self.config == 3:
                for p in self.model.expert_parameters():
                    p.grad *= self.expert_scale
        if self.low_mem:
            for p, m, o in zip(self.params, self.masters, self.opts):
                m.grad = p.grad.float()
                o.step()
                p.copy_(m)
                m.grad = None
            return
        if not self.fp32:
            torch._foreach_copy_([m.grad for m in self.masters], [p.grad for p in self.params])
        self.opt.step()
        if not self.fp32:
            torch._foreach_copy_(self.params, self.masters)

    @torch.no_grad()
    def _zero(self):
        for p in self.params:
            if p.grad is not None:
                p.grad.zero_()

    def _step_body(self):
        self._zero()
        loss = None
        for k in range(self.accum):
            if self.micro_feed is not None:
                self.micro_feed(k)
            loss = self._fwd_bwd()
        self._optim()
        self.loss.copy_(loss)

    def warm(self, n: int):
        # first steps eager (they create the gradient tensors), then try to capture
        for _ in range(max(n, 1)):
            self._step_body()
        torch.cuda.synchronize()
        if self.use_graph and self.micro_feed is None:
            try:
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g):
                    self._step_body()
                self.graph = g
                torch.cuda.synchronize()
            except Exception as e:       # capture is an optimisation of the baseline, not a requirement
                self.graph = None
                self.capture_error = repr(e)[:200]
                torch.cuda.synchronize()

    def step(self):
        if self.graph is not None:
            self.graph.replay()
        else:
            self._step_body()

    def executor(self) -> str:
        return "cuda graph replay" if self.graph is not None else "eager stream"
