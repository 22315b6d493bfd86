"""Device description, feature modules and device selection.

Parity: Source/Public/Oa/Runtime/Device.h (OaVkDeviceHardwareInfo / SoftwareInfo / DeviceInfo, the compute-device
queries), Device/DeviceBuilder.cpp (scoring and choosing a device by preference), Features/*.cpp (the Core / Ml / Vision /
Audio / Render feature modules and their trust gates) and the PCI-id performance table of DeviceUtils.cpp:315-392.
Here a device is a CUDA ordinal: the hardware record comes from the CUDA device properties, the performance figures from
the measured-peaks file when it is present (nominal B200 figures otherwise), and the feature gates answer what the
kernels of this package need: compute capability 10.x for the tcgen05 / TMEM / TMA paths, peer access for the fused
collectives.
"""
from __future__ import annotations

import enum
import json
import os
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Sequence

import torch

from ..core.types import OaStatus, OaStatusCode

NOMINAL_B200 = {"bf16_tflops": 2250.0, "hbm_gbs": 7700.0, "nvlink_gbs": 900.0, "sms": 148, "l2_mb": 126, "smem_kb": 227, "tmem_kb": 256,
                "hbm_gb": 180}


class OaDeviceType(enum.IntEnum):
    Cpu = 0
    DiscreteGpu = 1
    IntegratedGpu = 2


class OaFeatureModule(enum.IntFlag):
    Core = 1          # elementwise / reductions / fp32 paths
    Ml = 2            # tensor-core GEMM, attention, scans: needs tcgen05 + TMEM + TMA
    Vision = 4
    Audio = 8
    Crypto = 16
    Collective = 32   # fused compute + communication kernels over peer memory
    Render = 64       # needs a graphics stack: never offered here


@dataclass
class OaDeviceHardwareInfo:
    Ordinal: int = -1
    Name: str = "cpu"
    Type: OaDeviceType = OaDeviceType.Cpu
    ComputeMajor: int = 0
    ComputeMinor: int = 0
    MultiProcessorCount: int = 0
    TotalMemoryBytes: int = 0
    L2CacheBytes: int = 0
    SharedMemoryPerBlockOptin: int = 0
    PciBusId: str = ""

    def ComputeCapability(self) -> str: return f"{self.ComputeMajor}.{self.ComputeMinor}"
    def IsBlackwellDataCenter(self) -> bool: return self.ComputeMajor == 10


@dataclass
class OaDeviceSoftwareInfo:
    DriverVersion: str = ""
    CudaRuntime: str = ""
    TorchVersion: str = ""
    NcclVersion: str = ""
    KernelLibrary: str = ""
    Features: OaFeatureModule = OaFeatureModule(0)
    Reasons: Dict[str, str] = field(default_factory=dict)     # feature name -> why it is off


@dataclass
class OaDevicePerformance:
    Bf16Tflops: float = 0.0
    HbmGbs: float = 0.0
    Source: str = "none"          # "measured" | "nominal" | "none"


@dataclass
class OaDeviceInfo:
    Hardware: OaDeviceHardwareInfo = field(default_factory=OaDeviceHardwareInfo)
    Software: OaDeviceSoftwareInfo = field(default_factory=OaDeviceSoftwareInfo)
    Performance: OaDevicePerformance = field(default_factory=OaDevicePerformance)

    def Supports(self, module: OaFeatureModule) -> bool: return bool(self.Software.Features & module)

    def ToDict(self) -> dict:
        h, s, p = self.Hardware, self.Software, self.Performance
        return {"ordinal": h.Ordinal, "name": h.Name, "type": h.Type.name, "compute_capability": h.ComputeCapability(), "sms": h.MultiProcessorCount,
                "memory_gb": round(h.TotalMemoryBytes / 1e9, 1), "l2_mb": round(h.L2CacheBytes / 2 ** 20, 1), "driver": s.DriverVersion,
                "cuda": s.CudaRuntime, "features": [m.name for m in OaFeatureModule if s.Features & m], "feature_reasons": dict(s.Reasons),
                "bf16_tflops": p.Bf16Tflops, "hbm_gbs": p.HbmGbs, "performance_source": p.Source}


def LoadMeasuredPeaks(path: Optional[str] = None) -> Optional[dict]:
    """The measured copy bandwidth / GEMM throughput record of this pool, when the file exists."""
    cands = [path] if path else [os.environ.get("OA_MEASURED_PEAKS", ""), os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(
        os.path.abspath(__file__)))), "MEASURED_PEAKS.json")]
    for c in cands:
        if c and os.path.isfile(c):
            try:
                with open(c) as f:
                    return json.load(f)
            except (OSError, json.JSONDecodeError):
                return None
    return None


def _find(d, *names):
    """First numeric value stored under any of `names`, at any depth."""
    if isinstance(d, dict):
        for n in names:
            if isinstance(d.get(n), (int, float)):
                return float(d[n])
        for v in d.values():
            r = _find(v, *names)
            if r is not None:
                return r
    return None


def GateFeatures(hw: OaDeviceHardwareInfo, kernel_library_loaded: bool, peer_access: bool) -> OaDeviceSoftwareInfo:
    """Feature modules a device may run, with the reason for each one that is off."""
    sw = OaDeviceSoftwareInfo()
    feats, why = OaFeatureModule(0), {}
    if hw.Type == OaDeviceType.Cpu:
        feats = OaFeatureModule.Core | OaFeatureModule.Ml | OaFeatureModule.Vision | OaFeatureModule.Audio | OaFeatureModule.Crypto
        why["Collective"] = "CPU engine: collectives run through the process group"
    else:
        if not kernel_library_loaded:
            for m in ("Core", "Ml", "Vision", "Audio", "Crypto", "Collective"):
                why[m] = "the kernel library is not loaded"
        elif hw.ComputeMajor != 10:
            for m in ("Core", "Ml", "Vision", "Audio", "Crypto", "Collective"):
                why[m] = f"kernels are built for sm_100a only, the device is sm_{hw.ComputeMajor}{hw.ComputeMinor}"
        else:
            feats = OaFeatureModule.Core | OaFeatureModule.Ml | OaFeatureModule.Vision | OaFeatureModule.Audio | OaFeatureModule.Crypto
            if peer_access:
                feats |= OaFeatureModule.Collective
            else:
                why["Collective"] = "no peer access to another device"
    why["Render"] = "no graphics stack"
    sw.Features, sw.Reasons = feats, why
    return sw


def DescribeDevice(ordinal: int = 0, peaks: Optional[dict] = None) -> OaDeviceInfo:
    """Record of CUDA device `ordinal`, or of the host when no GPU is visible (or ordinal < 0)."""
    info = OaDeviceInfo()
    sw_common = dict(TorchVersion=torch.__version__, CudaRuntime=str(torch.version.cuda or ""))
    if ordinal < 0 or not torch.cuda.is_available() or ordinal >= torch.cuda.device_count():
        info.Software = GateFeatures(info.Hardware, False, False)
        for k, v in sw_common.items():
            setattr(info.Software, k, v)
        return info
    p = torch.cuda.get_device_properties(ordinal)
    info.Hardware = OaDeviceHardwareInfo(ordinal, p.name, OaDeviceType.IntegratedGpu if getattr(p, "is_integrated", 0) else OaDeviceType.DiscreteGpu,
                                         p.major, p.minor, p.multi_processor_count, p.total_memory, getattr(p, "L2_cache_size", 0),
                                         getattr(p, "shared_memory_per_block_optin", 0), getattr(p, "pci_bus_id", "") and str(p.pci_bus_id))
    from .. import _native as N
    peers = any(torch.cuda.can_device_access_peer(ordinal, o) for o in range(torch.cuda.device_count()) if o != ordinal)
    info.Software = GateFeatures(info.Hardware, N.lib() is not None, peers)
    for k, v in sw_common.items():
        setattr(info.Software, k, v)
    info.Software.KernelLibrary = str(N.lib_path())
    try:
        info.Software.NcclVersion = ".".join(str(x) for x in torch.cuda.nccl.version())
    except Exception:
        pass
    peaks = peaks if peaks is not None else LoadMeasuredPeaks()
    tf, bw = (_find(peaks, "bf16_tflops"), _find(peaks, "hbm_gbs")) if peaks else (None, None)
    if tf and bw:
        info.Performance = OaDevicePerformance(tf, bw, "measured")
    elif info.Hardware.IsBlackwellDataCenter():
        info.Performance = OaDevicePerformance(NOMINAL_B200["bf16_tflops"], NOMINAL_B200["hbm_gbs"], "nominal")
    return info


class OaDevicePreference(enum.IntEnum):
    Auto = 0
    HighPerformance = 1
    LowPower = 2
    Specific = 3


def ScoreDevice(info: OaDeviceInfo, preference: OaDevicePreference = OaDevicePreference.Auto) -> float:
    """Higher is better; a device that cannot run the ML module scores 0."""
    if not info.Supports(OaFeatureModule.Ml):
        return 0.0
    h = info.Hardware
    score = 1.0 + h.MultiProcessorCount * 10.0 + h.TotalMemoryBytes / 2 ** 30
    if h.Type == OaDeviceType.DiscreteGpu:
        score += 1000.0
    if info.Supports(OaFeatureModule.Collective):
        score += 100.0
    if preference == OaDevicePreference.LowPower:
        score = 1.0 + 1e6 / score
    return score


class OaDeviceBuilder:
    """Chooses a device: an explicit ordinal, else the best-scoring visible one, else the host."""

    def __init__(self, describe: Callable[[int], OaDeviceInfo] = DescribeDevice, count: Optional[Callable[[], int]] = None):
        self._describe = describe
        self._count = count or (lambda: torch.cuda.device_count() if torch.cuda.is_available() else 0)
        self.Preference, self.Ordinal = OaDevicePreference.Auto, -1
        self.Required = OaFeatureModule.Core

    def SetPreference(self, preference: OaDevicePreference, ordinal: int = -1) -> "OaDeviceBuilder":
        self.Preference, self.Ordinal = preference, ordinal
        return self

    def Require(self, modules: OaFeatureModule) -> "OaDeviceBuilder":
        self.Required = modules
        return self

    def Candidates(self) -> List[OaDeviceInfo]:
        return [self._describe(i) for i in range(self._count())]

    def Build(self):
        """(OaDeviceInfo, OaStatus)."""
        if self.Preference == OaDevicePreference.Specific:
            if not 0 <= self.Ordinal < self._count():
                return None, OaStatus(OaStatusCode.NotFound, f"no device with ordinal {self.Ordinal}")
            chosen = self._describe(self.Ordinal)
        else:
            ranked = sorted(self.Candidates(), key=lambda d: ScoreDevice(d, self.Preference), reverse=True)
            chosen = ranked[0] if ranked and ScoreDevice(ranked[0], self.Preference) > 0 else self._describe(-1)
        missing = [m.name for m in OaFeatureModule if (self.Required & m) and not chosen.Supports(m)]
        if missing:
            why = "; ".join(f"{m}: {chosen.Software.Reasons.get(m, 'not offered')}" for m in missing)
            return None, OaStatus(OaStatusCode.FailedPrecondition, f"{chosen.Hardware.Name} lacks {why}")
        return chosen, OaStatus.Ok()
