"""OaModule / OaParameter: the module tree, parameter registration and checkpoint walks.

Reference: Source/Public/Oa/Ml/Module.h:23-171, Source/Private/Oa/Ml/Nn/Module.cpp (save / validate / load walks
:150-321).  Names are dotted paths built from RegisterModule / RegisterParameter names; loading validates
name, dtype, rank, shape and byte count of EVERY tensor before any tensor is mutated.
"""
from __future__ import annotations

from typing import Optional

import torch

from ..core.matrix import OaMatrix
from ..core.types import OaError, OaStatus, OaStatusCode, from_torch_dtype
from ..io.oam import OamModel
from ..runtime import engine as RT


class OaParameter:
    def __init__(self, data: OaMatrix, name: str = "", requires_grad: bool = True):
        self.Data = data
        self.Name = name
        self.RequiresGrad = requires_grad
        data.SetRequiresGrad(requires_grad)
        data.Name = name

    def Grad(self) -> OaMatrix:
        return self.Data.GradMatrix()

    def Tensor(self) -> torch.Tensor:
        return self.Data.Tensor()

    def NumElements(self) -> int:
        return self.Data.NumElements()


class OaModuleBuffer:
    def __init__(self, data: OaMatrix, name: str, persistent: bool = True):
        self.Data = data
        self.Name = name
        self.Persistent = persistent


class OaNamedParameter:
    def __init__(self, name: str, param: OaParameter):
        self.Name = name
        self.Param = param


class OaModule:
    def __init__(self):
        self._params: list[OaParameter] = []
        self._buffers: list[OaModuleBuffer] = []
        self._children: list[tuple[str, "OaModule"]] = []
        self._training = True
        self._name = type(self).__name__

    # ---- forward
    def Forward(self, x: OaMatrix) -> OaMatrix:
        raise NotImplementedError(f"{type(self).__name__}.Forward")

    def __call__(self, *a, **k):
        return self.Forward(*a, **k)

    # ---- mode
    def Train(self, on: bool = True) -> "OaModule":
        self._training = on
        for _, c in self._children:
            c.Train(on)
        return self

    def Eval(self) -> "OaModule":
        return self.Train(False)

    def IsTraining(self) -> bool:
        return self._training

    class ScopedEval:
        def __init__(self, module: "OaModule"):
            self._m, self._prev = module, module.IsTraining()

        def __enter__(self):
            self._m.Eval()
            return self._m

        def __exit__(self, *a):
            self._m.Train(self._prev)
            return False

    # ---- registration
    def RegisterParameter(self, name: str, data: OaMatrix, requires_grad: bool = True) -> OaParameter:
        p = OaParameter(data, name, requires_grad)
        self._params.append(p)
        return p

    def RegisterModule(self, name: str, module: "OaModule") -> "OaModule":
        module.SetName(name)
        self._children.append((name, module))
        return module

    def RegisterBuffer(self, name: str, data: OaMatrix, persistent: bool = True) -> OaModuleBuffer:
        b = OaModuleBuffer(data, name, persistent)
        self._buffers.append(b)
        return b

    # ---- queries
    def Parameters(self) -> list[OaParameter]:
        """Parameters registered directly on this module (non-recursive)."""
        return self._params

    def Children(self):
        return self._children

    def Buffers(self):
        return self._buffers

    def AllNamedParameterPtrs(self, prefix: str = "") -> list[OaNamedParameter]:
        out = [OaNamedParameter(prefix + p.Name, p) for p in self._params]
        for name, c in self._children:
            out.extend(c.AllNamedParameterPtrs(prefix + name + "."))
        return out

    def AllParameterPtrs(self) -> list[OaParameter]:
        return [n.Param for n in self.AllNamedParameterPtrs()]

    AllParameters = AllParameterPtrs

    def AllBufferPtrs(self, persistent_only: bool = False, prefix: str = ""):
        out = [(prefix + b.Name, b) for b in self._buffers if b.Persistent or not persistent_only]
        for name, c in self._children:
            out.extend(c.AllBufferPtrs(persistent_only, prefix + name + "."))
        return out

    def NumParameters(self) -> int:
        return sum(p.NumElements() for p in self.AllParameterPtrs())

    def SetName(self, name: str) -> None:
        self._name = name

    def GetName(self) -> str:
        return self._name

    # ---- checkpoint
    def OamArchitecture(self) -> str:
        return type(self).__name__[:31]

    def SaveTo(self, oam: OamModel) -> OaStatus:
        RT.OaContext.GetDefault().Sync()
        wdt = None
        for n in self.AllNamedParameterPtrs():
            t = self._export_param(n.Name, n.Param)
            oam.AddWeight(n.Name, t)
            wdt = wdt or from_torch_dtype(t.dtype)
        for name, b in self.AllBufferPtrs(persistent_only=True):
            oam.AddState(name, b.Data.Tensor())
        cfg = self.OamConfig()
        oam.SetConfig(cfg.get("Architecture", self.OamArchitecture()), cfg.get("DModel", 0), cfg.get("NLayers", 0),
                      cfg.get("DVocab", 256), weight_dtype=wdt if wdt is not None else 0,
                      arch_config=cfg.get("ArchConfig", b""))
        return OaStatus.Ok()

    def OamConfig(self) -> dict:
        return {}

    def _export_param(self, name: str, p: OaParameter) -> torch.Tensor:
        """Hook for sharded parameters: return the canonical unsharded tensor."""
        return p.Tensor()

    def _import_param(self, name: str, p: OaParameter, host: torch.Tensor) -> None:
        p.Tensor().copy_(host.to(p.Tensor().device))

    def ValidateLoad(self, oam: OamModel) -> OaStatus:
        have = {w.Name: w for w in oam.Weights()}
        for n in self.AllNamedParameterPtrs():
            e = have.get(n.Name)
            if e is None:
                return OaStatus.Error(OaStatusCode.NotFound, f"checkpoint has no tensor '{n.Name}'")
            t = self._export_shape_dtype(n.Name, n.Param)
            if e.Dtype != from_torch_dtype(t[1]):
                return OaStatus.Error(OaStatusCode.InvalidArgument, f"dtype mismatch for '{n.Name}': file {e.Dtype.name}")
            if tuple(e.Shape) != tuple(t[0]):
                return OaStatus.Error(OaStatusCode.InvalidArgument,
                                      f"shape mismatch for '{n.Name}': file {tuple(e.Shape)} vs model {tuple(t[0])}")
        states = {s.Name: s for s in oam.States()}
        for name, b in self.AllBufferPtrs(persistent_only=True):
            e = states.get(name)
            if e is None:
                return OaStatus.Error(OaStatusCode.NotFound, f"checkpoint has no state '{name}'")
            if tuple(e.Shape) != tuple(b.Data.Tensor().shape):
                return OaStatus.Error(OaStatusCode.InvalidArgument, f"shape mismatch for state '{name}'")
        return OaStatus.Ok()

    def _export_shape_dtype(self, name: str, p: OaParameter):
        return tuple(p.Tensor().shape), p.Tensor().dtype

    def LoadFrom(self, oam: OamModel) -> OaStatus:
        st = self.ValidateLoad(oam)
        if not st:
            return st
        ctx = RT.OaContext.GetDefault()
        ctx.Execute()
        ctx.Sync()
        have = {w.Name: w for w in oam.Weights()}
        for n in self.AllNamedParameterPtrs():
            self._import_param(n.Name, n.Param, have[n.Name].ToTorch())
        states = {s.Name: s for s in oam.States()}
        for name, b in self.AllBufferPtrs(persistent_only=True):
            b.Data.Tensor().copy_(states[name].ToTorch().to(b.Data.Tensor().device))
        return OaStatus.Ok()

    def Save(self, path, optimizer=None) -> OaStatus:
        oam = OamModel()
        st = self.SaveTo(oam)
        if st and optimizer is not None:
            st = optimizer.SaveTo(oam)
        if not st:
            return st
        if optimizer is not None and hasattr(optimizer, "IsPrimaryWriter") and not optimizer.IsPrimaryWriter():
            return OaStatus.Ok()      # took part in the optimizer's gather; rank 0 writes the file
        return oam.Save(path)

    def Load(self, path, optimizer=None) -> OaStatus:
        oam, st = OamModel.Load(path)
        if not st:
            return st
        st = self.ValidateLoad(oam)
        if st and optimizer is not None:
            st = optimizer.ValidateLoad(oam)
        if not st:
            return st
        st = self.LoadFrom(oam)
        if st and optimizer is not None:
            st = optimizer.LoadFrom(oam)
        return st
