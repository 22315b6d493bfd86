"""OaFnLoss (Source/Public/Oa/Ml/FnLoss.h:11-98, Source/Private/Oa/Ml/FnLoss/FnLoss.cpp:177-479).

CrossEntropy is the mean over rows of `lse - logit[target]` with a per-row fp32 loss; an out-of-range
target makes that row (and so the mean) NaN.  The fused kernel also produces the logits gradient in the
forward pass (the reference registers the same fusion as CrossEntropyLossGradBwd).
"""
from __future__ import annotations

from typing import Optional

import torch

from ..core import fn_matrix as F
from ..core.matrix import OaMatrix
from ..ops import kernels as K
from . import autograd as AG

_last_name = ""


def LastName() -> str:
    return _last_name


def _set(name: str) -> None:
    global _last_name
    _last_name = name
    F._ctx_add(name)


def CrossEntropy(logits: OaMatrix, targets: OaMatrix, ignore_index: int = -100, in_place_grad: bool = False) -> OaMatrix:
    """Mean cross-entropy of [rows, vocab] logits against integer targets [rows].  The mean is over ALL rows (the
    reference's contract, Source/Private/Oa/Ml/FnLoss/FnLoss.cpp:177-260); a row whose target is `ignore_index` adds zero
    loss and zero gradient but still counts in the denominator - use MaskedCrossEntropy for a mean over the kept rows.

    With `in_place_grad` the logits buffer is overwritten by the gradient when autograd is recording
    (saves a [rows, vocab] allocation for large vocabularies); the caller must not read logits afterwards.
    """
    _set("CrossEntropy")
    lt = logits.Tensor()
    l2 = lt.reshape(-1, lt.shape[-1])
    rows = l2.shape[0]
    tg = targets.Tensor().reshape(-1)
    need = AG.IsEnabled() and logits.RequiresGrad()
    if need:
        row_loss, dl = K.xent_fwd_bwd(l2, tg, grad_scale=1.0 / rows, dlogits=l2 if in_place_grad else None,
                                      ignore_index=ignore_index)
    else:
        row_loss, dl = K.xent_fwd_bwd(l2, tg, ignore_index=ignore_index)
    out = OaMatrix(K.mean_f32(row_loss))

    def back(g):
        # g is the scalar upstream gradient (1.0 for a root loss)
        if g.numel() == 1 and g.dtype == torch.float32 and _is_one(g):
            return (dl.reshape(lt.shape), None)
        return (K.binary("mul", dl, g.reshape(1).to(dl.dtype)).reshape(lt.shape), None)

    return AG.attach("CrossEntropy", out, [logits, targets], back)


def _is_one(g: torch.Tensor) -> bool:
    # The tape seeds the root with ones_like(loss); recognise it without a device sync.
    return getattr(g, "_oa_root_seed", False)


def MaskedCrossEntropy(logits: OaMatrix, targets: OaMatrix, mask: OaMatrix) -> OaMatrix:
    """Cross-entropy averaged over rows whose mask is non-zero."""
    _set("MaskedCrossEntropy")
    tg = targets.Tensor().reshape(-1).clone()
    mk = mask.Tensor().reshape(-1)
    tg[mk == 0] = -100
    lt = logits.Tensor()
    l2 = lt.reshape(-1, lt.shape[-1])
    cnt = mk.ne(0).sum().clamp(min=1).float()
    need = AG.IsEnabled() and logits.RequiresGrad()
    row_loss, dl = K.xent_fwd_bwd(l2, tg, grad_scale=1.0 if need else None)
    out = OaMatrix((row_loss.sum() / cnt).reshape(1))
    return AG.attach("MaskedCrossEntropy", out, [logits, targets],
                     lambda g: ((dl.float() * (g.reshape(1) / cnt)).to(dl.dtype).reshape(lt.shape), None))


def CrossEntropyBwd(logits: OaMatrix, targets: OaMatrix) -> OaMatrix:
    l2 = logits.Tensor().reshape(-1, logits.Size(-1))
    _, dl = K.xent_fwd_bwd(l2, targets.Tensor().reshape(-1), grad_scale=1.0 / l2.shape[0])
    return OaMatrix(dl.reshape(logits.Tensor().shape))


def _elem_loss(name: str, pred: OaMatrix, target: OaMatrix, fwd, bwd) -> OaMatrix:
    _set(name)
    p, t = F._c(pred.Tensor()), F._c(target.Tensor())
    n = p.numel()
    per = fwd(p, t)
    out = OaMatrix(K.mean_f32(per if per.dtype == torch.float32 else K.cast(per, torch.float32)))
    return AG.attach(name, out, [pred, target], lambda g: (K.unary("scale", bwd(p, t), 1.0 / n) if _is_one(g) else
                                                           K.binary("mul", K.unary("scale", bwd(p, t), 1.0 / n), g.reshape(1).to(p.dtype)), None))


def Mse(pred, target):
    return _elem_loss("Mse", pred, target, lambda p, t: K.unary("square", K.binary("sub", p, t)),
                      lambda p, t: K.unary("scale", K.binary("sub", p, t), 2.0))


def L1(pred, target):
    return _elem_loss("L1", pred, target, lambda p, t: K.unary("abs", K.binary("sub", p, t)),
                      lambda p, t: K.unary("sign", K.binary("sub", p, t)))


def SmoothL1(pred, target, beta: float = 1.0):
    def fwd(p, t):
        d = K.unary("abs", K.binary("sub", p, t))
        quad = K.unary("scale", K.unary("square", d), 0.5 / beta)
        lin = K.unary("add_scalar", d, -0.5 * beta)
        return torch.where(d < beta, quad, lin)

    def bwd(p, t):
        d = K.binary("sub", p, t)
        return torch.where(d.abs() < beta, d / beta, torch.sign(d))

    return _elem_loss("SmoothL1", pred, target, fwd, bwd)


def Bce(pred, target, eps: float = 1e-7):
    def fwd(p, t):
        pc = p.clamp(eps, 1 - eps)
        return -(t * pc.log() + (1 - t) * (1 - pc).log())

    def bwd(p, t):
        pc = p.clamp(eps, 1 - eps)
        return (pc - t) / (pc * (1 - pc))

    return _elem_loss("Bce", pred, target, fwd, bwd)


def MseBwd(pred, target): return OaMatrix(K.unary("scale", K.binary("sub", F._c(pred.Tensor()), F._c(target.Tensor())), 2.0 / pred.NumElements()))
def L1Bwd(pred, target): return OaMatrix(K.unary("scale", K.unary("sign", K.binary("sub", F._c(pred.Tensor()), F._c(target.Tensor()))), 1.0 / pred.NumElements()))


def SmoothL1Bwd(pred, target, beta: float = 1.0):
    d = K.binary("sub", F._c(pred.Tensor()), F._c(target.Tensor()))
    return OaMatrix(torch.where(d.abs() < beta, d / beta, torch.sign(d)) / pred.NumElements())


def BceBwd(pred, target, eps: float = 1e-7):
    p, t = pred.Tensor().clamp(eps, 1 - eps), target.Tensor()
    return OaMatrix((p - t) / (p * (1 - p)) / pred.NumElements())
