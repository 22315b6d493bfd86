"""Mixture-of-experts primitives on raw tensors: fused router, expert plan, gather / combine and the grouped GEMMs.

CUDA tensors run the kernels of `csrc/kernels/moe.cu` and the grouped modes of the tcgen05 GEMM; CPU tensors run the
plain statement of the same math (also the oracle of the GPU tests).  Layout contract: routed rows are packed
expert-major, stable in token-major route order inside an expert, and every expert segment is padded to a multiple
of 128 rows (`offsets[e]` are the padded starts, `packed_token[r] == -1` marks padding).
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import _native as N
from . import kernels as K

SEG = 128


def max_rows(tokens: int, k: int, experts: int) -> int:
    """Static upper bound of the packed row count (dropless): routes plus worst-case padding, rounded to 128."""
    return (tokens * k + experts * (SEG - 1) + SEG - 1) // SEG * SEG


def topk(x: torch.Tensor, k: int):
    """Descending top-k of each row, ties to the lower index. Returns (values, int32 indices)."""
    idx = torch.sort(-x.float(), dim=1, stable=True).indices[:, :k]
    return torch.gather(x, 1, idx), idx.to(torch.int32)


def router(logits: torch.Tensor, k: int, sel_bias: Optional[torch.Tensor] = None):
    """probs = softmax(logits) fp32 [T,E]; idx = top-k of (logits + sel_bias) int32 [T,K]; w = renormalised probs [T,K]."""
    T, E = logits.shape
    probs = torch.empty((T, E), dtype=torch.float32, device=logits.device)
    idx = torch.empty((T, k), dtype=torch.int32, device=logits.device)
    w = torch.empty((T, k), dtype=torch.float32, device=logits.device)
    if not logits.is_cuda:
        lf = logits.float()
        p = torch.softmax(lf, -1)
        sel = lf + (sel_bias.float().reshape(1, E) if sel_bias is not None else 0)
        _, ii = topk(sel, k)
        pw = torch.gather(p, 1, ii.long())
        probs.copy_(p); idx.copy_(ii); w.copy_(pw / pw.sum(-1, keepdim=True))
        return probs, idx, w
    K._launch(N.require().oa_moe_router(K.dt(logits), logits.data_ptr(), N.ptr(sel_bias), probs.data_ptr(), idx.data_ptr(),
                                        w.data_ptr(), T, E, k, N.stream()), "oa_moe_router")
    return probs, idx, w


def router_bwd(probs, idx, w, dw, dprobs_col: Optional[torch.Tensor], dprobs_scale: float, out_dtype: torch.dtype):
    """dlogits [T,E] from the route-weight gradient dw [T,K] and an optional per-expert probability gradient
    (dprobs[t,e] = dprobs_col[e] * dprobs_scale, the form the load-balance loss produces)."""
    T, E = probs.shape
    k = idx.shape[1]
    dl = torch.empty((T, E), dtype=out_dtype, device=probs.device)
    if not probs.is_cuda:
        S = torch.gather(probs, 1, idx.long()).sum(-1, keepdim=True)
        dot = (dw * w).sum(-1, keepdim=True)
        dp = torch.zeros_like(probs)
        dp.scatter_add_(1, idx.long(), (dw - dot) / S)
        if dprobs_col is not None:
            dp = dp + dprobs_col.float().reshape(1, E) * dprobs_scale
        dl.copy_(probs * (dp - (dp * probs).sum(-1, keepdim=True)))
        return dl
    K._launch(N.require().oa_moe_router_bwd(K.dt(dl), probs.data_ptr(), idx.data_ptr(), w.data_ptr(), dw.data_ptr(),
                                            N.ptr(dprobs_col), float(dprobs_scale), dl.data_ptr(), T, E, k, N.stream()),
              "oa_moe_router_bwd")
    return dl


class Plan:
    __slots__ = ("counts", "offsets", "packed_token", "inverse", "max_rows", "experts", "k", "tokens")


def plan(idx: torch.Tensor, experts: int, rows_cap: Optional[int] = None) -> Plan:
    T, k = idx.shape
    P = Plan()
    P.experts, P.k, P.tokens = experts, k, T
    P.max_rows = rows_cap or max_rows(T, k, experts)
    dev = idx.device
    P.counts = torch.empty(experts, dtype=torch.int32, device=dev)
    P.offsets = torch.empty(experts + 1, dtype=torch.int32, device=dev)
    P.packed_token = torch.empty(P.max_rows, dtype=torch.int32, device=dev)
    P.inverse = torch.empty((T, k), dtype=torch.int32, device=dev)
    if not idx.is_cuda:
        flat = idx.reshape(-1).long()
        counts = torch.bincount(flat, minlength=experts)
        padded = (counts + SEG - 1) // SEG * SEG
        offs = torch.zeros(experts + 1, dtype=torch.long)
        offs[1:] = torch.cumsum(padded, 0)
        order = torch.sort(flat, stable=True).indices           # stable: route order kept inside an expert
        rank = torch.empty_like(order)
        start = torch.zeros(experts + 1, dtype=torch.long)
        start[1:] = torch.cumsum(counts, 0)
        rank[order] = torch.arange(order.numel()) - start[flat[order]]
        pos = offs[flat] + rank
        P.packed_token.fill_(-1)
        P.packed_token[pos] = (torch.arange(flat.numel()) // k).to(torch.int32)
        P.inverse.copy_(pos.reshape(T, k))
        P.counts.copy_(counts); P.offsets.copy_(offs)
        return P
    lib = N.require()
    sc = K.scratch(dev, lib.oa_moe_plan_scratch_bytes(T * k, experts), "moe_plan").view(torch.int32)
    K._launch(lib.oa_moe_plan(idx.data_ptr(), T, k, experts, P.counts.data_ptr(), P.offsets.data_ptr(), P.packed_token.data_ptr(),
                              P.inverse.data_ptr(), P.max_rows, sc.data_ptr(), N.stream()), "oa_moe_plan", 4)
    return P


def gather(x: torch.Tensor, P: Plan) -> torch.Tensor:
    """packed[r,:] = x[packed_token[r],:], zero for padding rows."""
    dim = x.shape[1]
    out = torch.empty((P.max_rows, dim), dtype=x.dtype, device=x.device)
    if not x.is_cuda:
        pt = P.packed_token.long()
        out.zero_()
        ok = pt >= 0
        out[ok] = x[pt[ok]]
        return out
    assert x.dtype == torch.bfloat16
    K._launch(N.require().oa_moe_gather(x.data_ptr(), P.packed_token.data_ptr(), out.data_ptr(), P.offsets.data_ptr(), P.experts,
                                        dim, P.max_rows, N.stream()), "oa_moe_gather")
    return out


def gather_bwd(dpacked: torch.Tensor, P: Plan, base: Optional[torch.Tensor] = None) -> torch.Tensor:
    dim = dpacked.shape[1]
    dx = torch.empty((P.tokens, dim), dtype=dpacked.dtype, device=dpacked.device)
    if not dpacked.is_cuda:
        inv = P.inverse.long()
        acc = base.float().clone() if base is not None else torch.zeros((P.tokens, dim))
        for kk in range(P.k):
            acc += dpacked.float()[inv[:, kk]]
        dx.copy_(acc)
        return dx
    K._launch(N.require().oa_moe_gather_bwd(dpacked.data_ptr(), P.inverse.data_ptr(), N.ptr(base), dx.data_ptr(), P.tokens, P.k, dim,
                                            N.stream()), "oa_moe_gather_bwd")
    return dx


def combine(packed: torch.Tensor, gate: torch.Tensor, P: Plan, base: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[t,:] = base[t,:] + sum_k gate[t,k] * packed[inverse[t,k],:]."""
    dim = packed.shape[1]
    out = torch.empty((P.tokens, dim), dtype=packed.dtype, device=packed.device)
    if not packed.is_cuda:
        inv = P.inverse.long()
        acc = base.float().clone() if base is not None else torch.zeros((P.tokens, dim))
        for kk in range(P.k):
            acc += gate[:, kk:kk + 1].float() * packed.float()[inv[:, kk]]
        out.copy_(acc)
        return out
    K._launch(N.require().oa_moe_combine(packed.data_ptr(), gate.data_ptr(), P.inverse.data_ptr(), N.ptr(base), out.data_ptr(),
                                         P.tokens, P.k, dim, N.stream()), "oa_moe_combine")
    return out


def combine_bwd(packed: torch.Tensor, gate: torch.Tensor, P: Plan, dout: torch.Tensor):
    """Returns (dpacked [max_rows, dim], dgate [T, K] fp32)."""
    dim = packed.shape[1]
    dpacked = torch.empty_like(packed)
    dgate = torch.zeros((P.tokens, P.k), dtype=torch.float32, device=packed.device)
    if not packed.is_cuda:
        inv = P.inverse.long()
        dpacked.zero_()
        for kk in range(P.k):
            dpacked[inv[:, kk]] = (gate[:, kk:kk + 1].float() * dout.float()).to(dpacked.dtype)
            dgate[:, kk] = (dout.float() * packed.float()[inv[:, kk]]).sum(-1)
        return dpacked, dgate
    K._launch(N.require().oa_moe_combine_bwd(packed.data_ptr(), gate.data_ptr(), P.inverse.data_ptr(), P.packed_token.data_ptr(),
                                             dout.data_ptr(), dpacked.data_ptr(), dgate.data_ptr(), P.offsets.data_ptr(), P.experts,
                                             P.k, dim, P.max_rows, N.stream()), "oa_moe_combine_bwd")
    return dpacked, dgate


def _segments(P: Plan):
    offs = P.offsets.tolist()
    return [(e, offs[e], offs[e + 1]) for e in range(P.experts)]


def grouped_linear(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], P: Plan, *, b_mn: bool = False,
                   act: int = K.ACT_NONE, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[r,:] = x[r,:] @ W[e(r)]^T (+ bias[e(r)]).  w is [E, N, K] (or [E, K, N] with b_mn: the data-gradient form)."""
    Nn = w.shape[2] if b_mn else w.shape[1]
    if out is None:
        out = torch.empty((P.max_rows, Nn), dtype=x.dtype, device=x.device)
    if not x.is_cuda:
        out.zero_()
        for e, lo, hi in _segments(P):
            if hi > lo:
                We = w[e].float()
                v = x[lo:hi].float() @ (We if b_mn else We.t())
                if bias is not None:
                    v = v + bias[e].float()
                out[lo:hi] = v
        return out
    assert x.dtype == torch.bfloat16 and w.is_contiguous()
    Kd = x.shape[1]
    K._launch(N.require().oa_gemm_bf16_grouped(1, x.data_ptr(), w.data_ptr(), out.data_ptr(), 0, Nn, Kd, x.stride(0), w.stride(1),
                                               out.stride(0), int(b_mn), N.ptr(bias), act, None, None, 0, 0, 0, P.experts,
                                               P.offsets.data_ptr(), P.max_rows, w.stride(0), 0,
                                               bias.stride(0) if bias is not None else 0, K.status_word(x.device).data_ptr(),
                                               N.stream()), "oa_gemm_bf16_grouped(rows)")
    return out


def grouped_weight_grad(dy: torch.Tensor, x: torch.Tensor, P: Plan, out: Optional[torch.Tensor] = None,
                        accumulate: bool = False) -> torch.Tensor:
    """dW[e] = dY_e^T @ X_e  ->  [E, N, K] for dy [rows, N], x [rows, K]."""
    Nn, Kd = dy.shape[1], x.shape[1]
    if out is None:
        out = torch.empty((P.experts, Nn, Kd), dtype=dy.dtype, device=dy.device)
    if not dy.is_cuda:
        for e, lo, hi in _segments(P):
            v = dy[lo:hi].float().t() @ x[lo:hi].float()
            out[e] = v + out[e].float() if accumulate else v
        return out
    K._launch(N.require().oa_gemm_bf16_grouped(2, dy.data_ptr(), x.data_ptr(), out.data_ptr(), Nn, Kd, 0, dy.stride(0), x.stride(0),
                                               out.stride(1), 0, None, K.ACT_NONE, None, None, 0, int(out.dtype == torch.float32),
                                               int(accumulate), P.experts, P.offsets.data_ptr(), P.max_rows, 0, out.stride(0), 0,
                                               K.status_word(dy.device).data_ptr(), N.stream()), "oa_gemm_bf16_grouped(reduce)")
    return out


def grouped_bias_grad(dy: torch.Tensor, P: Plan) -> torch.Tensor:
    """db[e] = column sums of dY over expert e's rows (padding rows are zero)."""
    Nn = dy.shape[1]
    out = torch.zeros((P.experts, Nn), dtype=dy.dtype, device=dy.device)
    offs = P.offsets.tolist() if not dy.is_cuda else None
    if offs is not None:
        for e in range(P.experts):
            out[e] = dy[offs[e]:offs[e + 1]].float().sum(0)
        return out
    # device path without a host sync: per-128-row block sums, then a segmented add by block -> expert map
    blocks = dy.reshape(P.max_rows // SEG, SEG, Nn)
    bsum = K.col_sum(K.contiguous(blocks.transpose(0, 1)).reshape(SEG, -1)).reshape(P.max_rows // SEG, Nn)
    starts = (P.offsets[:-1] // SEG).long()
    ends = (P.offsets[1:] // SEG).long()
    csum = torch.zeros((P.max_rows // SEG + 1, Nn), dtype=torch.float32, device=dy.device)
    csum[1:] = torch.cumsum(bsum.float(), 0)
    out.copy_(csum[ends] - csum[starts])
    return out
