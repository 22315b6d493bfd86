"""OaEngine / OaContext: device ownership and the record -> Execute -> Sync executor.

Reference: Source/Public/Oa/Runtime/Engine.h:83-546 (engine, config, modes),
Source/Public/Oa/Runtime/Context.h:46-155 (context facade), Source/Public/Oa/Runtime/Sync.h (events),
Source/Public/Oa/Runtime/GpuTimer.h:34-68.

B200 design: the reference records nodes into a Vulkan command graph and submits it at `Execute`.
Here an operation is enqueued on the context's CUDA stream when it is recorded (the stream *is* the
in-order command buffer), `Execute` closes the current recording interval, `Submit` returns an event
recorded on the stream and `Sync` waits for the stream and then checks the kernels' status word.
Results are therefore observable exactly where the reference makes them observable (after Sync/Wait),
while nothing is ever re-recorded: a whole training step is captured once into a CUDA graph by
`OaTrainingProgram` and replayed.  The context still keeps the node log (kernel name, buffers,
access) of the current interval for graph reports and hazard analysis.
"""
from __future__ import annotations

import enum
import os
import threading
import time
from dataclasses import dataclass, field
from typing import Optional

import torch

from ..core.types import OaError, OaNumericMode, OaPrecision, OaStatus, OaStatusCode
from ..utils import envflag


class OaDevicePreference(enum.IntEnum):
    Auto = 0
    Discrete = 1
    Integrated = 2
    Cpu = 3


class OaEngineState(enum.IntEnum):
    Empty = 0
    Initializing = 1
    Ready = 2
    Closing = 3
    Closed = 4
    Failed = 5


@dataclass
class OaEngineConfig:
    """Mirrors the fields of the reference's OaEngineConfig that have a meaning on CUDA."""

    DevicePreference: OaDevicePreference = OaDevicePreference.Auto
    DeviceIndex: int = -1                 # -1: LOCAL_RANK (or 0)
    Precision: OaPrecision = OaPrecision.FP32
    NumericMode: OaNumericMode = OaNumericMode.Fast
    EnableMultiDevice: bool = False
    MaxDevices: int = 8
    MeshDeviceIndices: list = field(default_factory=list)   # CUDA ordinals (reference: MeshVulkanIndices)
    EnableValidation: bool = False
    RecordGraph: bool = False             # keep the per-interval node log (graph reports)
    AppName: str = "oa_b200"


class OaEvent:
    """Completion token of a Submit(); engine provenance is checked on Wait (Runtime/Sync.h:60-108)."""

    def __init__(self, engine: "OaEngine", cuda_event=None):
        self._engine = engine
        self._ev = cuda_event
        self._done = cuda_event is None

    def IsComplete(self) -> bool:
        if self._done:
            return True
        self._done = bool(self._ev.query())
        return self._done

    def Wait(self) -> None:
        if not self._done:
            self._ev.synchronize()
            self._done = True


class OaGpuTimer:
    """Event pair around a region of the context's stream; ReadbackMs() blocks until the region finished."""

    def __init__(self, name: str = "timer"):
        self.Name = name
        eng = OaEngine.GetGlobal()
        self._cuda = torch.cuda.is_available() and (eng is None or eng.IsCuda())
        self._e0 = self._e1 = None
        self._t0 = self._t1 = 0.0

    def Begin(self) -> None:
        if self._cuda:
            self._e0 = torch.cuda.Event(enable_timing=True)
            self._e1 = torch.cuda.Event(enable_timing=True)
            self._e0.record()
        else:
            self._t0 = time.perf_counter()

    def End(self) -> None:
        if self._cuda:
            self._e1.record()
        else:
            self._t1 = time.perf_counter()

    def ReadbackMs(self) -> float:
        if self._cuda:
            if self._e1 is None:
                return 0.0
            self._e1.synchronize()
            return float(self._e0.elapsed_time(self._e1))
        return (self._t1 - self._t0) * 1e3


@dataclass
class OaExecutionStats:
    Nodes: int = 0
    Executes: int = 0
    Syncs: int = 0
    LastExecuteNodes: int = 0
    HostRecordMs: float = 0.0
    WaitMs: float = 0.0


class OaContext:
    """Recorder + executor bound to one CUDA stream (or to the CPU)."""

    _tls = threading.local()

    def __init__(self, engine: "OaEngine"):
        self._engine = engine
        self._stream = torch.cuda.Stream(device=engine.Device()) if engine.IsCuda() and envflag.IsSet("OA_OWN_STREAM") else None
        self._nodes: list = []
        self._interval_nodes = 0
        self._stats = OaExecutionStats()
        self._failure: Optional[OaStatus] = None
        self._recording = engine.Config.RecordGraph or envflag.IsSet("OA_GRAPH_REPORT")
        self._last_graph: list = []
        self._pending: Optional[OaEvent] = None

    # -- default context -------------------------------------------------
    @classmethod
    def GetDefault(cls) -> "OaContext":
        ctx = getattr(cls._tls, "ctx", None)
        eng = OaEngine.GetGlobal()
        if ctx is None or ctx._engine is not eng:
            if eng is None:
                eng = get_engine()          # lazily created with defaults, like every tensor factory does
            ctx = OaContext(eng)
            cls._tls.ctx = ctx
        return ctx

    # -- recording --------------------------------------------------------
    def Engine(self) -> "OaEngine":
        return self._engine

    def Stream(self):
        return self._stream if self._stream is not None else (torch.cuda.current_stream() if self._engine.IsCuda() else None)

    def Session(self):
        """The execution session of this context (stable resource frame, reusable graphs, batch hazards); created on
        first use so that contexts which never capture a step pay nothing."""
        if getattr(self, "_session", None) is None:
            from .session import OaExecutionSession
            self._session = OaExecutionSession(self._engine.Device())
        return self._session

    def Add(self, kernel: str, reads=(), writes=()) -> None:
        """Notes one recorded kernel node. Buffers are identified by their storage address."""
        self._interval_nodes += 1
        collecting = getattr(self, "_collect", None) is not None
        if self._recording or collecting:
            node = (kernel, tuple(_buf_id(t) for t in reads), tuple(_buf_id(t) for t in writes))
            if self._recording:
                self._nodes.append(node)
            if collecting:
                self._collect.append(node)

    def SetRecording(self, on: bool) -> None:
        self._recording = bool(on)

    # -- collection of one step for a training program (validate stage) ---------
    def BeginCollect(self) -> None:
        """Starts collecting the nodes of one recorded step (whatever the recording flag says) together with the marks
        of ops that cannot be replayed."""
        self._collect = []
        self._unsafe: list = []

    def EndCollect(self):
        """Returns (nodes, unsafe marks) of the step collected since BeginCollect."""
        nodes, unsafe = getattr(self, "_collect", None) or [], getattr(self, "_unsafe", [])
        self._collect = None
        return nodes, unsafe

    def IsCollecting(self) -> bool:
        return getattr(self, "_collect", None) is not None

    def MarkReplayUnsafe(self, reason: str) -> None:
        """An op calls this when it freezes a host-side value into its launch (a learning rate passed by value, a random
        offset, a host-computed count): a captured program that contains it would replay stale values, so capture is
        refused (Source/Private/Oa/Ml/TrainingProgram.cpp:167-252 rejects the same classes of node)."""
        if getattr(self, "_collect", None) is not None:
            self._unsafe.append(str(reason))

    @staticmethod
    def Compile(nodes):
        """Builds the native compute graph of a node list: hazards, dependency levels, alias groups, structural hash.
        Returns (OaComputeGraph, structure hash): the structure hash covers the kernel sequence only (buffer addresses
        differ between an eager step and a captured one), the graph's own hash covers buffers too."""
        from ..io.oam import OamHash
        from .graph import OaAccess, OaComputeGraph
        g = OaComputeGraph()
        for kernel, reads, writes in nodes:
            bufs = [(b, 0, OaAccess.Read) for b in reads] + [(b, 0, OaAccess.Write) for b in writes]
            g.AddNode(kernel, bufs)
        return g, OamHash("\n".join(n[0] for n in nodes).encode())

    def RecordFailure(self, status: OaStatus) -> None:
        """Sticky recording failure: surfaces at the next Execute and clears the interval (rollback)."""
        if self._failure is None:
            self._failure = status

    def NodeCount(self) -> int:
        return self._interval_nodes

    # -- execution --------------------------------------------------------
    def Execute(self) -> OaStatus:
        if self._failure is not None:
            st, self._failure = self._failure, None
            self.Clear()
            return st
        self._stats.Executes += 1
        self._stats.Nodes += self._interval_nodes
        self._stats.LastExecuteNodes = self._interval_nodes
        if self._recording:
            self._last_graph = self._nodes
            # the interval as the native compute graph sees it: hazards, dependency levels, structural hash
            graph, structure = OaContext.Compile(self._nodes)
            self._last_compiled = {"nodes": len(self._nodes), "levels": graph.NumLevels(), "barriers": graph.NumBarriers(),
                                   "hash": graph.Hash(), "structure_hash": structure}
        self._nodes = []
        self._interval_nodes = 0
        return OaStatus.Ok()

    def Submit(self, timer: Optional[OaGpuTimer] = None) -> OaEvent:
        st = self.Execute()
        if not st:
            raise OaError(st)
        if timer is not None:
            timer.End()
        if self._engine.IsCuda():
            ev = torch.cuda.Event()
            ev.record(self.Stream())
            self._pending = OaEvent(self._engine, ev)
        else:
            self._pending = OaEvent(self._engine, None)
        return self._pending

    def Wait(self, event: OaEvent) -> OaStatus:
        if event._engine is not self._engine:
            return OaStatus.Error(OaStatusCode.InvalidArgument, "event belongs to another engine")
        t0 = time.perf_counter()
        event.Wait()
        self._stats.WaitMs += (time.perf_counter() - t0) * 1e3
        return self._check_device()

    def Sync(self) -> OaStatus:
        self._stats.Syncs += 1
        if self._engine.IsCuda():
            t0 = time.perf_counter()
            s = self.Stream()
            if not torch.cuda.is_current_stream_capturing():
                s.synchronize()
            self._stats.WaitMs += (time.perf_counter() - t0) * 1e3
            return self._check_device()
        return OaStatus.Ok()

    def _check_device(self) -> OaStatus:
        from ..ops import kernels as K
        if not self._engine.IsCuda():
            return OaStatus.Ok()
        try:
            if not torch.cuda.is_current_stream_capturing():
                K.check_status(self._engine.Device())
        except Exception as e:  # a bounded device wait ran out
            return OaStatus.Error(OaStatusCode.DeadlineExceeded, str(e))
        return OaStatus.Ok()

    def Clear(self) -> None:
        self._nodes = []
        self._interval_nodes = 0

    def LastExecutionStats(self) -> OaExecutionStats:
        return self._stats

    def LastGraph(self) -> list:
        return list(self._last_graph)

    def LastCompiled(self) -> dict:
        """Report of the native compute graph of the last executed interval (recording must be on)."""
        return dict(getattr(self, "_last_compiled", {}))

    def MaxAsyncSubmissions(self) -> int:
        return 1

    # context-manager form used by the Python surface: executes and syncs on exit
    def __enter__(self):
        return self

    def __exit__(self, exc_type, exc, tb):
        if exc_type is None:
            st = self.Execute()
            if st:
                st = self.Sync()
            if not st:
                raise OaError(st)
        return False


def _buf_id(t) -> int:
    try:
        return t.untyped_storage().data_ptr()
    except Exception:
        return id(t)


class OaEngine:
    """Owner of the device, the default stream, the parallel mesh and process-wide numeric settings."""

    _global: Optional["OaEngine"] = None
    _lock = threading.Lock()

    def __init__(self):
        self.Config = OaEngineConfig()
        self.State = OaEngineState.Empty
        self._device = torch.device("cpu")
        self._weight_dtype = torch.float32
        self.Mesh = None

    # -- life cycle -------------------------------------------------------
    @classmethod
    def Create(cls, config: Optional[OaEngineConfig] = None) -> "OaEngine":
        eng = cls()
        st = eng.InitInPlace(config or OaEngineConfig())
        if not st:
            raise OaError(st)
        return eng

    def InitInPlace(self, config: OaEngineConfig) -> OaStatus:
        self.State = OaEngineState.Initializing
        self.Config = config
        forced = envflag.GetString("OA_FORCE_PRECISION", "")
        if forced:
            config.Precision = OaPrecision.BF16 if forced.lower() in ("bf16", "bfloat16") else OaPrecision.FP32
        if envflag.IsSet("OA_DISABLE_BF16"):
            config.Precision = OaPrecision.FP32
        want_cpu = config.DevicePreference == OaDevicePreference.Cpu or envflag.GetString("OA_DEVICE", "") == "cpu"
        if torch.cuda.is_available() and not want_cpu:
            idx = config.DeviceIndex
            if idx < 0:
                idx = envflag.GetInt("OA_DEVICE", -1)
            if idx < 0:
                idx = int(os.environ.get("LOCAL_RANK", "0"))
            if idx >= torch.cuda.device_count():
                self.State = OaEngineState.Failed
                return OaStatus.Error(OaStatusCode.NotFound, f"CUDA device {idx} not present")
            self._device = torch.device("cuda", idx)
            torch.cuda.set_device(self._device)
            from .. import _native
            _native.require()  # a GPU box without the kernel library is an error, never a fallback
        else:
            self._device = torch.device("cpu")
        self._weight_dtype = torch.bfloat16 if config.Precision == OaPrecision.BF16 else torch.float32
        if config.NumericMode == OaNumericMode.Deterministic:
            os.environ.setdefault("OA_DETERMINISTIC", "1")
        self.State = OaEngineState.Ready
        return OaStatus.Ok()

    def SetAsGlobal(self) -> None:
        with OaEngine._lock:
            OaEngine._global = self

    @classmethod
    def GetGlobal(cls) -> Optional["OaEngine"]:
        return cls._global

    def Close(self) -> None:
        if self.State in (OaEngineState.Closed, OaEngineState.Empty):
            return
        self.State = OaEngineState.Closing
        if self.IsCuda():
            torch.cuda.synchronize(self._device)
        if self.Mesh is not None:
            self.Mesh.Close()
            self.Mesh = None
        with OaEngine._lock:
            if OaEngine._global is self:
                OaEngine._global = None
        self.State = OaEngineState.Closed

    # -- queries ----------------------------------------------------------
    def IsInitialized(self) -> bool:
        return self.State == OaEngineState.Ready

    def Device(self) -> torch.device:
        return self._device

    def IsCuda(self) -> bool:
        return self._device.type == "cuda"

    def Precision(self) -> OaPrecision:
        return self.Config.Precision

    def WeightDtype(self) -> torch.dtype:
        return self._weight_dtype

    def SetWeightDtype(self, dtype: torch.dtype) -> None:
        self._weight_dtype = dtype

    def IsBlackwell(self) -> bool:
        return self.IsCuda() and torch.cuda.get_device_capability(self._device)[0] >= 10

    def DeviceName(self) -> str:
        return torch.cuda.get_device_name(self._device) if self.IsCuda() else "cpu"

    # -- buffers (Engine.h:274-281) ----------------------------------------
    def AllocateBuffer(self, nbytes: int) -> torch.Tensor:
        return torch.empty(int(nbytes), dtype=torch.uint8, device=self._device)

    def UploadBuffer(self, dst: torch.Tensor, src_bytes) -> None:
        host = torch.frombuffer(bytearray(src_bytes), dtype=torch.uint8)
        dst.view(torch.uint8).reshape(-1)[: host.numel()].copy_(host, non_blocking=False)

    def ReadbackBuffer(self, src: torch.Tensor) -> bytes:
        if self.IsCuda():
            torch.cuda.current_stream().synchronize()
        return src.detach().contiguous().view(torch.uint8).cpu().numpy().tobytes()


def OaInitComputeEngine(config: Optional[OaEngineConfig] = None) -> bool:
    """Creates (once) the process-wide engine. Importing the package never does this implicitly."""
    if OaEngine.GetGlobal() is not None and OaEngine.GetGlobal().IsInitialized():
        return True
    try:
        eng = OaEngine.Create(config)
    except OaError:
        return False
    eng.SetAsGlobal()
    from .gemm_tuner import InstallFromEnv
    InstallFromEnv()                      # OA_GEMM_TUNE / OA_GEMM_PLANS: launch plans of the GEMM family from the native plan cache
    return True


def OaShutdownComputeEngine() -> None:
    eng = OaEngine.GetGlobal()
    if eng is not None:
        eng.Close()


def OaContextGetDefault() -> OaContext:
    return OaContext.GetDefault()


def get_engine() -> OaEngine:
    """The global engine; created lazily with defaults (the reference's Python module does the same)."""
    eng = OaEngine.GetGlobal()
    if eng is None:
        if not OaInitComputeEngine():
            raise OaError(OaStatus.Error(OaStatusCode.Unavailable, "compute engine initialisation failed"))
        eng = OaEngine.GetGlobal()
    return eng
