"""Block-level fused operations used by the Transformer layers.

The reference plans such fusions in its DNN planner (engines `PackedQkv`, `GatedFfn`, `ResidualNorm`,
Source/Public/Oa/Runtime/Dnn.h:16-100).  Here each is one autograd node whose forward and backward use the
GEMM epilogues (bias, GELU, residual add, GELU-backward) so that no separate elementwise pass touches the
[tokens, ffn] activations.
"""
from __future__ import annotations

from typing import Optional, Sequence

import torch

from ..core import fn_matrix as F
from ..core.matrix import OaMatrix
from ..ops import kernels as K
from . import autograd as AG


def packed_view(tensors: Sequence[torch.Tensor]) -> Optional[torch.Tensor]:
    """If the given row-major tensors sit back to back in one storage, returns them as one tensor
    (rows concatenated); otherwise None.  Parameters registered together end up adjacent in the
    optimizer's flat arena, which is what makes packed QKV / gate-up projections copy-free."""
    t0 = tensors[0]
    if not all(t.is_contiguous() and t.dtype == t0.dtype and t.shape[1:] == t0.shape[1:] for t in tensors):
        return None
    st = t0.untyped_storage()
    ptr = t0.data_ptr()
    for t in tensors:
        if t.untyped_storage().data_ptr() != st.data_ptr() or t.data_ptr() != ptr:
            return None
        ptr += t.numel() * t.element_size()
    rows = sum(t.shape[0] for t in tensors)
    return torch.empty(0, dtype=t0.dtype, device=t0.device).set_(st, t0.storage_offset(), (rows, *t0.shape[1:]))


def _packed_param(params: Sequence[OaMatrix]):
    """(weight view, grad view or None) for adjacent parameters, or (None, None)."""
    w = packed_view([p.Tensor() for p in params])
    if w is None:
        return None, None
    grads = [p.GradTensor() for p in params]
    g = packed_view(grads) if all(x is not None for x in grads) else None
    return w, g


def _sink_state(params: Sequence[OaMatrix]):
    """Consumes the 'fresh' flags of a group of leaves; returns accumulate (True if any already holds a gradient)."""
    acc = False
    for p in params:
        s = p.GradSink()
        if s is not None and s[1]:
            acc = True
    return acc


def PackedProjection(x: OaMatrix, weights: Sequence[OaMatrix], biases: Sequence[Optional[OaMatrix]], name: str = "PackedLinear") -> OaMatrix:
    """y[M, sum N_i] = x @ [W_0; W_1; ...]^T (+ [b_0; b_1; ...]) as ONE GEMM.  Uses the storage adjacency of the
    parameters when present and falls back to concatenating copies (reference: PackedLinear2/3)."""
    has_bias = all(b is not None for b in biases) and len(biases) > 0
    w, gw = _packed_param(weights)
    b, gb = _packed_param(biases) if has_bias else (None, None)
    if w is None or (has_bias and b is None):
        return F.PackedLinear(x, list(weights), list(biases))
    F._ctx_add(name)
    tx = x.Tensor()
    x2 = F._rows(tx)
    y = K.gemm(x2, w, bias=b)
    out = OaMatrix(y.reshape(*tx.shape[:-1], w.shape[0]))

    def back(g):
        g2 = F._rows(g)
        dx = K.gemm(g2, w, b_mn=True).reshape(tx.shape) if x.RequiresGrad() else None
        res = [dx]
        if gw is not None and all(p.IsLeaf() for p in weights):
            K.gemm(g2, x2, a_mn=True, b_mn=True, out=gw, accumulate=_sink_state(weights))
            res += [None] * len(weights)
        else:
            dw = K.gemm(g2, x2, a_mn=True, b_mn=True)
            o = 0
            for p in weights:
                res.append(dw[o:o + p.Size(0)])
                o += p.Size(0)
        if has_bias:
            if gb is not None and all(p.IsLeaf() for p in biases):
                K.col_sum(g2, out=gb, accumulate=_sink_state(biases))
                res += [None] * len(biases)
            else:
                db = K.col_sum(g2)
                o = 0
                for p in biases:
                    res.append(db[o:o + p.Size(0)])
                    o += p.Size(0)
        return tuple(res)

    ins = [x] + list(weights) + (list(biases) if has_bias else [])
    return AG.attach(name, out, ins, back)


def FfnGelu(x: OaMatrix, w1: OaMatrix, b1: Optional[OaMatrix], w2: OaMatrix, b2: Optional[OaMatrix],
            residual: Optional[OaMatrix] = None, act: int = K.ACT_GELU) -> OaMatrix:
    """y = act(x W1^T + b1) W2^T + b2 (+ residual).  Backward computes dz = (dy W2) * act'(z) inside the GEMM epilogue."""
    F._ctx_add("LinearGelu")
    F._ctx_add("Linear")
    tx = x.Tensor()
    x2 = F._rows(tx)
    tw1, tw2 = F._c(w1.Tensor()), F._c(w2.Tensor())
    z = torch.empty((x2.shape[0], tw1.shape[0]), dtype=tx.dtype, device=tx.device)
    h = K.gemm(x2, tw1, bias=b1.Tensor() if b1 is not None else None, act=act, aux_out=z)
    res2 = F._rows(residual.Tensor()) if residual is not None else None
    y = K.gemm(h, tw2, bias=b2.Tensor() if b2 is not None else None, residual=res2)
    out = OaMatrix(y.reshape(*tx.shape[:-1], tw2.shape[0]))
    bwd_act = K.ACT_GELU_BWD if act == K.ACT_GELU else K.ACT_RELU_BWD

    def back(g):
        g2 = F._rows(g)
        dz = K.gemm(g2, tw2, b_mn=True, act=bwd_act, aux_in=z)
        dw2 = _weight_grad(w2, g2, h)
        db2 = F._bias_grad(b2, g2)
        dw1 = _weight_grad(w1, dz, x2)
        db1 = F._bias_grad(b1, dz)
        dx = K.gemm(dz, tw1, b_mn=True).reshape(tx.shape) if x.RequiresGrad() else None
        return (dx, dw1, db1, dw2, db2, g if residual is not None else None)

    return AG.attach("FfnGelu", out, [x, w1, b1, w2, b2, residual], back)


def _weight_grad(w: OaMatrix, g2: torch.Tensor, x2: torch.Tensor):
    if w is None or not w.RequiresGrad():
        return None
    tw = w.Tensor()
    buf, acc, direct = F._grad_out(w, tw.shape, tw.dtype, tw.device)
    K.gemm(g2, x2, a_mn=True, b_mn=True, out=buf, accumulate=acc)
    return None if direct else buf


def FfnSwiglu(x: OaMatrix, gate_w: OaMatrix, up_w: OaMatrix, down_w: OaMatrix, residual: Optional[OaMatrix] = None) -> OaMatrix:
    """y = (silu(x Wg^T) * (x Wu^T)) Wd^T (+ residual); gate and up run as one packed GEMM."""
    gu = PackedProjection(x, [gate_w, up_w], [None, None], "PackedLinear2")
    h = F.Swiglu(gu)
    return F.Linear(h, down_w, None, residual=residual)
