"""OamModel: Python face of the native `.oam` reader / writer (`csrc/runtime/oam.cpp`).

Format and semantics: Source/Public/Oa/Ml/Oam.h:22-244, Source/Private/Oa/Ml/Oam.cpp (save :320-481, load :485-...).
Files written here are laid out byte-for-byte like the reference's (section order, page alignment,
FNV-1a payload checksums and the manifest checksum), so checkpoints are interchangeable.
"""
from __future__ import annotations

import ctypes
from pathlib import Path
from typing import Optional

import numpy as np
import torch

from ..core.types import OaScalarType, OaStatus, OaStatusCode, from_torch_dtype, to_torch_dtype

_LIB_PATH = Path(__file__).resolve().parent.parent / "_lib" / "liboa_runtime.so"
_lib: Optional[ctypes.CDLL] = None

u8p, u64p, f32p = ctypes.POINTER(ctypes.c_uint8), ctypes.POINTER(ctypes.c_uint64), ctypes.POINTER(ctypes.c_float)


def runtime_lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not _LIB_PATH.exists():
            from .. import build
            build.build_runtime()
        L = ctypes.CDLL(str(_LIB_PATH))
        L.oam_create.restype = ctypes.c_void_p
        L.oam_load.restype = ctypes.c_void_p
        L.oam_load.argtypes = [ctypes.c_char_p]
        L.oam_destroy.argtypes = [ctypes.c_void_p]
        L.oam_last_error.restype = ctypes.c_char_p
        L.oam_hash.restype = ctypes.c_uint64
        L.oam_hash.argtypes = [ctypes.c_char_p, ctypes.c_uint64]
        L.oam_save.argtypes = [ctypes.c_void_p, ctypes.c_char_p]
        L.oam_set_config.argtypes = [ctypes.c_void_p, ctypes.c_char_p, ctypes.c_uint32, ctypes.c_uint32, ctypes.c_uint32,
                                     ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_uint32, ctypes.c_char_p, ctypes.c_uint64]
        L.oam_get_config.argtypes = [ctypes.c_void_p, ctypes.c_char_p, ctypes.POINTER(ctypes.c_uint32), ctypes.POINTER(ctypes.c_uint32),
                                     ctypes.POINTER(ctypes.c_uint32), ctypes.POINTER(ctypes.c_int), ctypes.POINTER(ctypes.c_uint32)]
        L.oam_arch_config.restype = ctypes.c_uint64
        L.oam_arch_config.argtypes = [ctypes.c_void_p, ctypes.POINTER(u8p)]
        L.oam_format_version.restype = ctypes.c_uint32
        L.oam_format_version.argtypes = [ctypes.c_void_p]
        L.oam_add_tensor.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_char_p, ctypes.c_int, ctypes.c_int, u64p,
                                     ctypes.c_void_p, ctypes.c_uint64]
        L.oam_num_tensors.restype = ctypes.c_uint32
        L.oam_num_tensors.argtypes = [ctypes.c_void_p, ctypes.c_int]
        L.oam_tensor_at.restype = ctypes.c_void_p
        L.oam_tensor_at.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_uint32, ctypes.c_char_p, ctypes.POINTER(ctypes.c_int),
                                    ctypes.POINTER(ctypes.c_int), u64p, u64p]
        L.oam_set_optimizer.argtypes = [ctypes.c_void_p, ctypes.c_char_p, ctypes.c_float, ctypes.c_float, ctypes.c_float,
                                        ctypes.c_float, ctypes.c_float, ctypes.c_int64, ctypes.c_void_p, ctypes.c_uint64,
                                        ctypes.c_void_p, ctypes.c_uint64, ctypes.c_void_p, ctypes.c_uint64]
        L.oam_has_optimizer.argtypes = [ctypes.c_void_p]
        L.oam_get_optimizer.argtypes = [ctypes.c_void_p, ctypes.c_char_p, f32p, ctypes.POINTER(ctypes.c_int64), u64p,
                                        ctypes.POINTER(f32p), ctypes.POINTER(f32p), ctypes.POINTER(f32p)]
        L.oam_set_progress.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int64, ctypes.c_uint64, ctypes.c_uint64,
                                       ctypes.c_float, ctypes.c_float, ctypes.c_int, ctypes.c_char_p]
        L.oam_get_progress.argtypes = [ctypes.c_void_p, ctypes.POINTER(ctypes.c_int), ctypes.POINTER(ctypes.c_int64), u64p, u64p,
                                       f32p, f32p, ctypes.POINTER(ctypes.c_int), ctypes.c_char_p]
        _lib = L
    return _lib


def OamHash(data: bytes) -> int:
    return int(runtime_lib().oam_hash(data, len(data)))


class OamTensor:
    __slots__ = ("Name", "Dtype", "Shape", "NumBytes", "_ptr", "_owner")

    def ToTorch(self) -> torch.Tensor:
        """Host tensor copy of the payload."""
        buf = (ctypes.c_uint8 * self.NumBytes).from_address(self._ptr) if self.NumBytes else b""
        raw = torch.frombuffer(bytearray(buf), dtype=torch.uint8) if self.NumBytes else torch.empty(0, dtype=torch.uint8)
        return raw.view(to_torch_dtype(self.Dtype)).reshape(self.Shape).clone()


class OamOptimizerState:
    def __init__(self):
        self.Type = "AdamW"
        self.Lr, self.Beta1, self.Beta2, self.Eps, self.WeightDecay = 3e-4, 0.9, 0.999, 1e-8, 0.1
        self.Step = 0
        self.AdamM = np.zeros(0, np.float32)
        self.AdamV = np.zeros(0, np.float32)
        self.MuonM = np.zeros(0, np.float32)


class OamProgress:
    def __init__(self):
        self.Phase, self.Step, self.BytesSeen, self.EnvSteps = 0, 0, 0, 0
        self.Lr, self.BestMetric, self.LowerIsBetter, self.MetricName = 3e-4, 0.0, True, "loss"


class OamModel:
    """In-memory model file: config, weight / state tensors, optimizer state, progress."""

    def __init__(self, handle: Optional[int] = None):
        self._L = runtime_lib()
        self._h = handle if handle is not None else self._L.oam_create()
        self._keep = []

    def __del__(self):
        try:
            if self._h:
                self._L.oam_destroy(self._h)
                self._h = None
        except Exception:
            pass

    # ---- config
    def SetConfig(self, architecture: str, d_model: int = 0, n_layers: int = 0, d_vocab: int = 256,
                  weight_dtype=OaScalarType.Float32, state_dtype=OaScalarType.Float32, compute_dtype=OaScalarType.Float32,
                  flags: int = 0, arch_config: bytes = b"") -> None:
        self._L.oam_set_config(self._h, architecture.encode(), d_model, n_layers, d_vocab, int(weight_dtype), int(state_dtype),
                               int(compute_dtype), flags, arch_config, len(arch_config))

    def GetConfig(self) -> dict:
        arch = ctypes.create_string_buffer(32)
        dm, nl, dv, fl = ctypes.c_uint32(), ctypes.c_uint32(), ctypes.c_uint32(), ctypes.c_uint32()
        dts = (ctypes.c_int * 3)()
        self._L.oam_get_config(self._h, arch, ctypes.byref(dm), ctypes.byref(nl), ctypes.byref(dv), dts, ctypes.byref(fl))
        p = u8p()
        n = self._L.oam_arch_config(self._h, ctypes.byref(p))
        return {"Architecture": arch.value.decode(), "DModel": dm.value, "NLayers": nl.value, "DVocab": dv.value,
                "WeightDtype": OaScalarType(dts[0]), "StateDtype": OaScalarType(dts[1]), "ComputeDtype": OaScalarType(dts[2]),
                "Flags": fl.value, "ArchConfig": bytes(ctypes.string_at(p, n)) if n else b""}

    def FormatVersion(self) -> int:
        return int(self._L.oam_format_version(self._h))

    # ---- tensors
    def _add(self, is_state: int, name: str, t: torch.Tensor) -> None:
        if len(name.encode()) > 127:
            raise ValueError(f"tensor name too long for .oam: {name}")
        host = t.detach().contiguous().cpu()
        dtype = from_torch_dtype(host.dtype)
        shape = (ctypes.c_uint64 * 8)(*list(host.shape) + [0] * (8 - host.dim()))
        raw = host.view(torch.uint8) if host.numel() else host
        nbytes = host.numel() * host.element_size()
        self._L.oam_add_tensor(self._h, is_state, name.encode(), int(dtype), host.dim(), shape,
                               raw.data_ptr() if nbytes else None, nbytes)

    def AddWeight(self, name: str, t: torch.Tensor) -> None:
        self._add(0, name, t)

    def AddState(self, name: str, t: torch.Tensor) -> None:
        self._add(1, name, t)

    def _tensors(self, is_state: int):
        out = []
        for i in range(self._L.oam_num_tensors(self._h, is_state)):
            name = ctypes.create_string_buffer(128)
            dt, rk, nb = ctypes.c_int(), ctypes.c_int(), ctypes.c_uint64()
            shape = (ctypes.c_uint64 * 8)()
            ptr = self._L.oam_tensor_at(self._h, is_state, i, name, ctypes.byref(dt), ctypes.byref(rk), shape, ctypes.byref(nb))
            e = OamTensor()
            e.Name, e.Dtype, e.Shape, e.NumBytes, e._ptr, e._owner = (name.value.decode(), OaScalarType(dt.value),
                                                                     tuple(int(shape[k]) for k in range(rk.value)), int(nb.value), ptr, self)
            out.append(e)
        return out

    def Weights(self):
        return self._tensors(0)

    def States(self):
        return self._tensors(1)

    def FindWeight(self, name: str) -> Optional[OamTensor]:
        for e in self.Weights():
            if e.Name == name:
                return e
        return None

    def FindState(self, name: str) -> Optional[OamTensor]:
        for e in self.States():
            if e.Name == name:
                return e
        return None

    def HasWeights(self) -> bool:
        return self._L.oam_num_tensors(self._h, 0) > 0

    # ---- optimizer / progress
    def SetOptimizer(self, st: OamOptimizerState) -> None:
        m = np.ascontiguousarray(st.AdamM, np.float32)
        v = np.ascontiguousarray(st.AdamV, np.float32)
        mu = np.ascontiguousarray(st.MuonM, np.float32)
        self._L.oam_set_optimizer(self._h, st.Type.encode(), st.Lr, st.Beta1, st.Beta2, st.Eps, st.WeightDecay, int(st.Step),
                                  m.ctypes.data, m.size, v.ctypes.data, v.size, mu.ctypes.data, mu.size)

    def HasOptimizer(self) -> bool:
        return bool(self._L.oam_has_optimizer(self._h))

    def GetOptimizer(self) -> OamOptimizerState:
        ty = ctypes.create_string_buffer(16)
        hy = (ctypes.c_float * 5)()
        step = ctypes.c_int64()
        counts = (ctypes.c_uint64 * 3)()
        pm, pv, pmu = f32p(), f32p(), f32p()
        self._L.oam_get_optimizer(self._h, ty, hy, ctypes.byref(step), counts, ctypes.byref(pm), ctypes.byref(pv), ctypes.byref(pmu))
        st = OamOptimizerState()
        st.Type = ty.value.decode()
        st.Lr, st.Beta1, st.Beta2, st.Eps, st.WeightDecay = (float(hy[i]) for i in range(5))
        st.Step = int(step.value)
        st.AdamM = np.ctypeslib.as_array(pm, (counts[0],)).copy() if counts[0] else np.zeros(0, np.float32)
        st.AdamV = np.ctypeslib.as_array(pv, (counts[1],)).copy() if counts[1] else np.zeros(0, np.float32)
        st.MuonM = np.ctypeslib.as_array(pmu, (counts[2],)).copy() if counts[2] else np.zeros(0, np.float32)
        return st

    def SetProgress(self, p: OamProgress) -> None:
        self._L.oam_set_progress(self._h, p.Phase, p.Step, p.BytesSeen, p.EnvSteps, p.Lr, p.BestMetric, int(p.LowerIsBetter),
                                 p.MetricName.encode())

    def GetProgress(self) -> OamProgress:
        ph, lo = ctypes.c_int(), ctypes.c_int()
        step = ctypes.c_int64()
        bs, es = ctypes.c_uint64(), ctypes.c_uint64()
        lr, best = ctypes.c_float(), ctypes.c_float()
        name = ctypes.create_string_buffer(32)
        self._L.oam_get_progress(self._h, ctypes.byref(ph), ctypes.byref(step), ctypes.byref(bs), ctypes.byref(es), ctypes.byref(lr),
                                 ctypes.byref(best), ctypes.byref(lo), name)
        p = OamProgress()
        p.Phase, p.Step, p.BytesSeen, p.EnvSteps = ph.value, step.value, bs.value, es.value
        p.Lr, p.BestMetric, p.LowerIsBetter, p.MetricName = lr.value, best.value, bool(lo.value), name.value.decode()
        return p

    # ---- file IO
    def Save(self, path) -> OaStatus:
        rc = self._L.oam_save(self._h, str(path).encode())
        if rc != 0:
            return OaStatus.Error(OaStatusCode(rc) if rc in OaStatusCode._value2member_map_ else OaStatusCode.Unknown,
                                  self._L.oam_last_error().decode())
        return OaStatus.Ok()

    @staticmethod
    def Load(path):
        """Returns (OamModel | None, OaStatus)."""
        L = runtime_lib()
        h = L.oam_load(str(path).encode())
        if not h:
            msg = L.oam_last_error().decode()
            code = OaStatusCode.DataLoss if msg.startswith("corrupt") else OaStatusCode.NotFound
            return None, OaStatus.Error(code, msg)
        return OamModel(h), OaStatus.Ok()
