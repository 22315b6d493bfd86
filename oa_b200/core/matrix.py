"""OaMatrix: value-semantic tensor handle with optional autograd meta.

Reference: Source/Public/Oa/Core/Matrix.h:21-211 (handle, views, operators, gradient accessors) and
Source/Python/Core/Type.cpp:71-155 (the Python method set).  Storage, allocator and dtype come from
`torch.Tensor`; every arithmetic method goes through `OaFnMatrix`, i.e. through this package's kernels.
"""
from __future__ import annotations

from typing import Optional, Sequence

import torch

from .types import OaMatrixShape, OaScalarType, from_torch_dtype, to_torch_dtype


class _AutogradMeta:
    __slots__ = ("requires_grad", "grad_fn", "grad", "grad_fresh")

    def __init__(self):
        self.requires_grad = False
        self.grad_fn = None
        self.grad = None          # torch.Tensor (persistent for parameters)
        self.grad_fresh = True    # True: next accumulation overwrites (set by ZeroGrad)


class OaMatrix:
    __slots__ = ("_t", "_meta", "Name")

    def __init__(self, tensor: Optional[torch.Tensor] = None):
        self._t = tensor
        self._meta: Optional[_AutogradMeta] = None
        self.Name = ""

    # ---- raw access -------------------------------------------------------
    def Tensor(self) -> torch.Tensor:
        return self._t

    # ---- shape / dtype ----------------------------------------------------
    def IsEmpty(self) -> bool:
        return self._t is None or self._t.numel() == 0

    def Rank(self) -> int:
        return 0 if self._t is None else self._t.dim()

    def NumElements(self) -> int:
        return 0 if self._t is None else self._t.numel()

    def ByteSize(self) -> int:
        return 0 if self._t is None else self._t.numel() * self._t.element_size()

    def Size(self, dim: int) -> int:
        return self._t.shape[dim]

    def Shape(self) -> OaMatrixShape:
        return OaMatrixShape(self._t.shape) if self._t is not None else OaMatrixShape()

    GetShape = Shape

    def Dtype(self) -> OaScalarType:
        return from_torch_dtype(self._t.dtype)

    GetDtype = Dtype

    def DeviceIndex(self) -> int:
        return self._t.device.index if self._t.is_cuda else -1

    # ---- views / copies (differentiable through OaFnMatrix) ----------------
    def Reshape(self, shape: Sequence[int]) -> "OaMatrix":
        from . import fn_matrix as F
        return F.Reshape(self, shape)

    View = Reshape

    def Flatten(self) -> "OaMatrix":
        return self.Reshape([self.NumElements()])

    def Unsqueeze(self, dim: int) -> "OaMatrix":
        s = list(self._t.shape)
        if dim < 0:
            dim += len(s) + 1
        s.insert(dim, 1)
        return self.Reshape(s)

    def Squeeze(self, dim: Optional[int] = None) -> "OaMatrix":
        s = list(self._t.shape)
        if dim is None:
            s = [d for d in s if d != 1]
        elif s[dim] == 1:
            s.pop(dim)
        return self.Reshape(s)

    def Transpose(self, d0: int = 0, d1: int = 1) -> "OaMatrix":
        from . import fn_matrix as F
        return F.Transpose(self, d0, d1)

    def Permute(self, dims: Sequence[int]) -> "OaMatrix":
        from . import fn_matrix as F
        return F.Permute(self, dims)

    def Contiguous(self) -> "OaMatrix":
        from ..ops import kernels as K
        if self._t.is_contiguous():
            return self
        return OaMatrix(K.contiguous(self._t))

    def Clone(self) -> "OaMatrix":
        from ..ops import kernels as K
        t = self._t if self._t.is_contiguous() else K.contiguous(self._t)
        if t.dtype in (torch.float32, torch.bfloat16):
            return OaMatrix(K.unary("copy", t))
        return OaMatrix(t.clone())

    def Detach(self) -> "OaMatrix":
        return OaMatrix(self._t)

    def CopyFrom(self, other: "OaMatrix") -> None:
        self._t.copy_(other._t)

    def To(self, device) -> "OaMatrix":
        """Copy to another device of the mesh (peer-to-peer when both are CUDA devices)."""
        dev = device if isinstance(device, torch.device) else torch.device("cuda", int(device))
        return OaMatrix(self._t.to(dev, non_blocking=True))

    def Zero(self) -> None:
        from ..ops import kernels as K
        K.fill_(self._t, 0.0)

    # ---- host access (synchronising) --------------------------------------
    def Item(self) -> float:
        return float(self._t.reshape(-1)[0].item())

    def At(self, *idx: int) -> float:
        if len(idx) == 1 and self._t.dim() != 1:
            return float(self._t.reshape(-1)[idx[0]].item())
        return float(self._t[tuple(idx)].item())

    def Set(self, *args) -> None:
        *idx, value = args
        if len(idx) == 1 and self._t.dim() != 1:
            self._t.reshape(-1)[idx[0]] = value
        else:
            self._t[tuple(idx)] = value

    def CopyToHost(self):
        return self._t.detach().float().cpu().reshape(-1).tolist()

    def __int__(self) -> int:
        return int(self._t.reshape(-1)[0].item())

    def __float__(self) -> float:
        return self.Item()

    # ---- autograd ----------------------------------------------------------
    def _meta_or_new(self) -> _AutogradMeta:
        if self._meta is None:
            self._meta = _AutogradMeta()
        return self._meta

    def RequiresGrad(self) -> bool:
        return self._meta is not None and self._meta.requires_grad

    def SetRequiresGrad(self, on: bool = True) -> "OaMatrix":
        self._meta_or_new().requires_grad = bool(on)
        return self

    def GetGradFn(self):
        return self._meta.grad_fn if self._meta is not None else None

    def _set_grad_fn(self, node) -> None:
        m = self._meta_or_new()
        m.grad_fn = node
        m.requires_grad = True

    def HasGradFn(self) -> bool:
        return self.GetGradFn() is not None

    def IsLeaf(self) -> bool:
        return self.GetGradFn() is None

    def GradMatrix(self) -> "OaMatrix":
        m = self._meta
        return OaMatrix(m.grad) if m is not None and m.grad is not None else OaMatrix()

    MutGradMatrix = GradMatrix

    def GradTensor(self) -> Optional[torch.Tensor]:
        return self._meta.grad if self._meta is not None else None

    def SetGradBuffer(self, buf: torch.Tensor) -> None:
        """Installs a persistent gradient buffer (e.g. a view of a flat gradient arena)."""
        m = self._meta_or_new()
        m.grad = buf
        m.grad_fresh = True

    def GradSink(self):
        """(buffer, accumulate) when a kernel may write this leaf's gradient directly, else None."""
        m = self._meta
        if m is None or m.grad is None or m.grad_fn is not None:
            return None
        acc = not m.grad_fresh
        m.grad_fresh = False
        return m.grad, acc

    def AccumulateGradTensor(self, d: torch.Tensor) -> None:
        from ..ops import kernels as K
        m = self._meta_or_new()
        if m.grad is None:
            m.grad = d if d.is_contiguous() else K.contiguous(d)
            m.grad_fresh = False
            return
        d = d.reshape(m.grad.shape)
        if m.grad_fresh:
            if d.dtype == m.grad.dtype and d.is_contiguous() and d.dtype in (torch.float32, torch.bfloat16):
                K.unary("copy", d, out=m.grad)
            else:
                K.cast(d, m.grad.dtype, out=m.grad)
            m.grad_fresh = False
        else:
            K.binary("add", m.grad, d if d.dtype == m.grad.dtype else K.cast(d, m.grad.dtype), out=m.grad)

    def AccumulateGrad(self, d: "OaMatrix") -> None:
        self.AccumulateGradTensor(d._t)

    def ZeroGrad(self) -> None:
        from ..ops import kernels as K
        m = self._meta
        if m is not None and m.grad is not None:
            K.fill_(m.grad, 0.0)
            m.grad_fresh = True

    def _mark_grad_fresh(self) -> None:
        """The owner of the gradient buffer zeroed it already (flat arena): the next accumulation overwrites."""
        m = self._meta
        if m is not None and m.grad is not None:
            m.grad_fresh = True

    # ---- operators -----------------------------------------------------------
    def _bin(self, other, name, scalar_name=None, reverse=False):
        from . import fn_matrix as F
        if isinstance(other, OaMatrix):
            return getattr(F, name)(other, self) if reverse else getattr(F, name)(self, other)
        return getattr(F, scalar_name)(self, float(other))

    def __add__(self, o): return self._bin(o, "Add", "AddScalar")
    def __radd__(self, o): return self._bin(o, "Add", "AddScalar")
    def __sub__(self, o): return self._bin(o, "Sub", "SubScalar")
    def __mul__(self, o): return self._bin(o, "Mul", "Scale")
    def __rmul__(self, o): return self._bin(o, "Mul", "Scale")
    def __truediv__(self, o): return self._bin(o, "Div", "DivScalar")

    def __rsub__(self, o):
        from . import fn_matrix as F
        return F.AddScalar(F.Neg(self), float(o))

    def __neg__(self):
        from . import fn_matrix as F
        return F.Neg(self)

    def __iadd__(self, o):
        r = self + o
        self._t, self._meta = r._t, r._meta
        return self

    def __isub__(self, o):
        r = self - o
        self._t, self._meta = r._t, r._meta
        return self

    def __imul__(self, o):
        r = self * o
        self._t, self._meta = r._t, r._meta
        return self

    def __itruediv__(self, o):
        r = self / o
        self._t, self._meta = r._t, r._meta
        return self

    def __repr__(self) -> str:
        if self._t is None:
            return "OaMatrix(empty)"
        return f"OaMatrix(shape={tuple(self._t.shape)}, dtype={self.Dtype().name}, device={self._t.device})"
