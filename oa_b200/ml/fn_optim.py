"""OaFnOptim: stateless optimizer steps over matrices (Source/Public/Oa/Ml/FnOptim.h:16-117).

The optimizer classes of `ml/optim.py` run the same kernels over flat arenas; these functions are the per-tensor
functional surface of the reference: `AdamWStep`, `AdamWAdvanceGraphState`, `AdamWStepGraph`, `AdamWStepMany`,
`AdamWStepManyGraph`, `SgdStep`, `MuonStep`, `ClipGradNorm`.  Every function records one node in the active OaContext and
mutates its in/out arguments in place.

Replay-safe ("Graph") variants read their scalars from a device state instead of launch arguments, so a captured step
keeps following `SetLr` and advances its own step counter.  The state here is float32[8]
{step, lr, beta1, beta2, eps, weight_decay, grad_scale, unused} (`MakeAdamWState`); the reference packs the same six
scalars as bit-cast uint32[6].
"""
from __future__ import annotations

from typing import NamedTuple, Optional, Sequence

import torch

from ..core.matrix import OaMatrix
from ..ops import kernels as K
from ..runtime import engine as RT


class OaAdamWParamSet(NamedTuple):
    Param: OaMatrix
    M: OaMatrix
    V: OaMatrix
    Grad: OaMatrix


def _t(m) -> torch.Tensor:
    return m.Tensor() if isinstance(m, OaMatrix) else m


def _flat(m) -> torch.Tensor:
    t = _t(m)
    assert t.is_contiguous(), "optimizer steps work on contiguous matrices"
    return t.view(-1)


def MakeAdamWState(step: int, lr: float, beta1: float = 0.9, beta2: float = 0.999, eps: float = 1e-8, weight_decay: float = 0.01,
                   grad_scale: float = 1.0, device=None) -> OaMatrix:
    """Device state of the replay-safe AdamW ops; `step` is the number of COMPLETED steps (AdamWAdvanceGraphState adds one
    right before the updates of the next step)."""
    dev = device or RT.get_engine().Device()
    return OaMatrix(torch.tensor([float(step), lr, beta1, beta2, eps, weight_decay, grad_scale, 0.0], dtype=torch.float32, device=dev))


def AdamWAdvanceGraphState(state) -> None:
    """state[0] += 1 on the device (one thread): each replay of a captured step consumes a distinct optimizer step."""
    RT.OaContext.GetDefault().Add("AdamwGraphAdvance")
    K.optim_advance(_t(state))


def AdamWStepGraph(param, m, v, grad, state, master: Optional[OaMatrix] = None) -> None:
    """AdamW with every scalar read from `state` (its step already advanced)."""
    RT.OaContext.GetDefault().Add("AdamwGraph")
    K.adam_step(_flat(param), _flat(grad), _flat(master) if master is not None else None, _flat(m), _flat(v), _t(state),
                decoupled=True)


def AdamWStep(param, m, v, grad, lr: float, beta1: float, beta2: float, eps: float, weight_decay: float, step: int,
              master: Optional[OaMatrix] = None) -> None:
    """param -= lr * (m_hat / (sqrt(v_hat) + eps) + weight_decay * param); `step` is the 1-based step being taken."""
    ctx = RT.OaContext.GetDefault()
    ctx.MarkReplayUnsafe("OaFnOptim.AdamWStep passes its scalars as launch arguments: use AdamWStepGraph inside a captured step")
    ctx.Add("Adamw")
    p = _flat(param)
    state = torch.tensor([float(step), lr, beta1, beta2, eps, weight_decay, 1.0, 0.0], dtype=torch.float32, device=p.device)
    K.adam_step(p, _flat(grad), _flat(master) if master is not None else None, _flat(m), _flat(v), state, decoupled=True)


def AdamWStepMany(params: Sequence[OaAdamWParamSet], lr: float, beta1: float, beta2: float, eps: float, weight_decay: float,
                  step: int) -> None:
    """AdamWStep over several parameter tensors with one shared scalar state."""
    if not params:
        return
    ctx = RT.OaContext.GetDefault()
    ctx.MarkReplayUnsafe("OaFnOptim.AdamWStepMany passes its scalars as launch arguments: use AdamWStepManyGraph inside a captured step")
    dev = _t(params[0].Param).device
    state = torch.tensor([float(step), lr, beta1, beta2, eps, weight_decay, 1.0, 0.0], dtype=torch.float32, device=dev)
    for s in params:
        ctx.Add("AdamwMany")
        K.adam_step(_flat(s.Param), _flat(s.Grad), None, _flat(s.M), _flat(s.V), state, decoupled=True)


def AdamWStepManyGraph(params: Sequence[OaAdamWParamSet], state) -> None:
    ctx = RT.OaContext.GetDefault()
    for s in params:
        ctx.Add("AdamwManyGraph")
        K.adam_step(_flat(s.Param), _flat(s.Grad), None, _flat(s.M), _flat(s.V), _t(state), decoupled=True)


def SgdStep(param, momentum, grad, lr: float, momentum_coef: float, weight_decay: float) -> None:
    """m = mu * m + g; param -= lr * m + weight_decay * param (decay not scaled by lr, as the reference's SgdMomentum).
    Pass `momentum=None` (or a coefficient of 0) for plain SGD."""
    ctx = RT.OaContext.GetDefault()
    ctx.MarkReplayUnsafe("OaFnOptim.SgdStep passes its scalars as launch arguments")
    use_mom = momentum is not None and momentum_coef != 0.0 and _t(momentum).numel() > 0
    ctx.Add("SgdMomentum" if use_mom else "Sgd")
    K.sgd_step(_flat(param), _flat(grad), None, _flat(momentum) if use_mom else None, lr=float(lr), momentum=float(momentum_coef),
               weight_decay=float(weight_decay))


def MuonStep(param, momentum, grad, lr: float, beta: float, weight_decay: float, eps: float = 1e-7, ns5_iterations: int = 5) -> None:
    """Muon: Nesterov momentum, Newton-Schulz-5 orthogonalisation of 2-D updates with the 0.2 * sqrt(max dim) scale,
    decoupled weight decay; 1-D parameters take the momentum update as it is."""
    from .optim import MoonshotScale, NewtonSchulz5
    ctx = RT.OaContext.GetDefault()
    ctx.MarkReplayUnsafe("OaFnOptim.MuonStep applies host-side scalars")
    p, mom, g = _t(param), _flat(momentum), _flat(grad).float()
    ctx.Add("MuonNesterov")
    mom.mul_(beta).add_(g, alpha=1 - beta)
    nest = g * (1 - beta) + mom * beta
    w = p.view(-1)
    if p.dim() == 2:
        rows, cols = p.shape
        ctx.Add("MuonNormalize")
        ortho = NewtonSchulz5(nest.view(rows, cols), int(ns5_iterations), float(eps)).reshape(-1)
        ctx.Add("MuonApply")
        upd = ortho * (-lr * MoonshotScale(rows, cols))
    else:
        ctx.Add("MuonVector")
        upd = nest * (-lr)
    w32 = w.float().mul_(1 - lr * weight_decay).add_(upd)
    w.copy_(w32)


def ClipGradNorm(grads: Sequence, max_norm: float, scratch_params=None, scratch_partials=None) -> OaMatrix:
    """Scales every gradient by min(1, max_norm / ||all grads||) on the device, no host synchronisation.  The two scratch
    arguments of the reference (persistent uint[17] / float[16] buffers) are accepted; the partial buffer, when given,
    holds {sum of squares, coefficient} afterwards.  Returns the 1-element coefficient matrix."""
    ctx = RT.OaContext.GetDefault()
    live = [g for g in grads if g is not None and _t(g).numel() > 0]
    if len(live) > 16:
        raise ValueError("ClipGradNorm takes at most 16 gradient matrices")
    dev = _t(live[0]).device if live else RT.get_engine().Device()
    buf = _t(scratch_partials) if scratch_partials is not None else torch.zeros(16, dtype=torch.float32, device=dev)
    assert buf.dtype == torch.float32 and buf.numel() >= 2
    ctx.Add("ClipGradNormReduce")
    if not live:
        buf[0:2] = torch.tensor([0.0, 1.0], device=buf.device)
        return OaMatrix(buf[1:2])
    for i, g in enumerate(live):
        K.sumsq(_flat(g), buf[0:1], accumulate=i > 0)
    K.clip_coef(buf[0:1], float(max_norm), buf[1:2])
    ctx.Add("ClipGradNormScale")
    for g in live:
        K.scale_inplace(_flat(g), buf[1:2])
    return OaMatrix(buf[1:2])
