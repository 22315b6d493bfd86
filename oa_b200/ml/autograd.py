"""Reverse-mode autograd tape (Source/Public/Oa/Ml/Autograd.h:12-96,
Source/Private/Oa/Ml/Autograd/Core/AutogradCore.cpp:17-202).

Thread-local enable flag and sequence counter; `OaGradientTape.Backward` collects the nodes reachable
from the root, orders them by sequence number, walks them in reverse, normalises view-shaped upstream
gradients, accumulates into leaves, adds fan-out contributions and releases saved tensors as soon as a
node has run.  Nodes work on raw tensors and launch the backward kernels on the context's stream.
"""
from __future__ import annotations

import threading
from typing import Callable, Optional, Sequence

import torch

_tls = threading.local()


def IsEnabled() -> bool:
    return getattr(_tls, "enabled", False)


def SetEnabled(on: bool) -> None:
    _tls.enabled = bool(on)


def NextSeq() -> int:
    n = getattr(_tls, "seq", 0) + 1
    _tls.seq = n
    return n


# A data-parallel wrapper overlaps its gradient reduction with the rest of the backward pass: it registers a hook that is
# called (a) when a backward pass starts and (b) each time a leaf has received its LAST gradient contribution of the pass.
_leaf_ready_hook = None
_backward_begin_hook = None


def SetLeafReadyHooks(on_begin, on_leaf_ready) -> None:
    """on_begin() at the start of every Backward; on_leaf_ready(matrix) when no node of the pass still writes to the leaf's
    gradient.  Pass (None, None) to remove them."""
    global _leaf_ready_hook, _backward_begin_hook
    _backward_begin_hook, _leaf_ready_hook = on_begin, on_leaf_ready


class OaGradNode:
    """One recorded differentiable operation.

    `backward(upstream: Tensor) -> sequence of (Tensor | None)` returns one gradient per graph input.
    With `fold = i` the node takes `backward(upstream, pending)`: `pending` is the gradient that input i has already
    collected from its other consumers (or None) and the returned gradient of input i then CONTAINS it, so the pass
    replaces the pending gradient instead of launching an add (a norm under a residual stream folds the stream's
    gradient into its own backward kernel).
    """

    __slots__ = ("name", "inputs", "backward", "seq", "out_shape", "saved", "fold")

    def __init__(self, name: str, inputs: Sequence, backward: Callable, out_shape, fold: Optional[int] = None):
        self.name = name
        self.inputs = list(inputs)
        self.backward = backward
        self.seq = NextSeq()
        self.out_shape = tuple(out_shape)
        self.saved = None
        self.fold = fold

    def GraphInputs(self):
        return self.inputs

    def ClearTensors(self) -> None:
        self.inputs = []
        self.backward = None
        self.saved = None


class OaGradNo:
    """Scope with autograd recording switched off."""

    def __enter__(self):
        self._prev = IsEnabled()
        SetEnabled(False)
        return self

    def __exit__(self, *a):
        SetEnabled(self._prev)
        return False


class OaGradientTape:
    """Scope with autograd recording on; `Backward(root)` records the backward kernels."""

    def __init__(self):
        self._prev = IsEnabled()
        self._active = True
        SetEnabled(True)

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.Close()
        return False

    def Close(self) -> None:
        if self._active:
            SetEnabled(self._prev)
            self._active = False

    def Backward(self, root, grad: Optional[torch.Tensor] = None) -> None:
        from ..ops import kernels as K

        if grad is None and root.NumElements() != 1:
            raise ValueError("backward root must be a scalar")
        root_fn = root.GetGradFn()
        if root_fn is None:
            return
        topo, seen, stack = [], set(), [root_fn]
        while stack:
            fn = stack.pop()
            if id(fn) in seen:
                continue
            seen.add(id(fn))
            topo.append(fn)
            for inp in fn.inputs:
                child = inp.GetGradFn() if inp is not None else None
                if child is not None and id(child) not in seen:
                    stack.append(child)
        topo.sort(key=lambda n: n.seq)
        hook = _leaf_ready_hook
        pending = None
        if hook is not None:
            if _backward_begin_hook is not None:
                _backward_begin_hook()
            pending = {}
            for fn in topo:
                for inp in fn.inputs:
                    if inp is not None and inp.IsLeaf() and inp.RequiresGrad():
                        e = pending.get(id(inp))
                        if e is None:
                            pending[id(inp)] = [1, inp]
                        else:
                            e[0] += 1
        if grad is None:
            grad = torch.ones_like(root.Tensor())
            grad._oa_root_seed = True   # lets scalar losses skip the multiply by 1 without reading the device
        grad_map = {id(root_fn): grad}
        with OaGradNo():
            for fn in reversed(topo):
                up = grad_map.pop(id(fn), None)
                if up is None:
                    if pending is not None:
                        _count_down(fn, pending, hook)
                    continue
                if tuple(up.shape) != fn.out_shape and up.numel() == _numel(fn.out_shape):
                    up = up.reshape(fn.out_shape)
                folded = None
                if fn.fold is None:
                    in_grads = fn.backward(up)
                else:
                    fi = fn.inputs[fn.fold]
                    fchild = fi.GetGradFn() if (fi is not None and not fi.IsLeaf() and fi.RequiresGrad()) else None
                    if fchild is not None:
                        prev = grad_map.get(id(fchild))
                        ft = fi.Tensor()
                        if prev is not None and tuple(prev.shape) == tuple(ft.shape) and prev.dtype == ft.dtype:
                            folded = prev
                    in_grads = fn.backward(up, folded)
                for idx, (inp, d) in enumerate(zip(fn.inputs, in_grads)):
                    if inp is None or d is None or not inp.RequiresGrad():
                        continue
                    if tuple(d.shape) != tuple(inp.Tensor().shape) and d.numel() == inp.NumElements():
                        d = d.reshape(inp.Tensor().shape)
                    if inp.IsLeaf():
                        inp.AccumulateGradTensor(d)
                        continue
                    child = inp.GetGradFn()
                    if child is None:
                        continue
                    prev = grad_map.get(id(child))
                    if prev is None or (folded is not None and idx == fn.fold):
                        grad_map[id(child)] = d            # first contribution, or one that already contains the pending gradient
                    else:
                        if tuple(d.shape) != tuple(prev.shape):
                            d = d.reshape(prev.shape)
                        grad_map[id(child)] = K.binary("add", prev, d if d.dtype == prev.dtype else d.to(prev.dtype))
                if pending is not None:
                    _count_down(fn, pending, hook)
                fn.ClearTensors()


def _count_down(fn, pending, hook) -> None:
    """`fn` has run (or was skipped): every leaf it feeds has one contribution less to wait for."""
    for inp in fn.inputs:
        if inp is None:
            continue
        e = pending.get(id(inp))
        if e is None:
            continue
        e[0] -= 1
        if e[0] == 0:
            del pending[id(inp)]
            hook(e[1])


def _numel(shape) -> int:
    n = 1
    for d in shape:
        n *= d
    return n


def attach(name: str, out, inputs: Sequence, backward: Callable, fold: Optional[int] = None):
    """Attaches a grad node to `out` when recording is on and some input needs a gradient (`fold`: see OaGradNode)."""
    if not IsEnabled():
        return out
    need = False
    for i in inputs:
        if i is not None and i.RequiresGrad():
            need = True
            break
    if not need:
        return out
    node = OaGradNode(name, inputs, backward, out.Tensor().shape, fold)
    out._set_grad_fn(node)
    return out
