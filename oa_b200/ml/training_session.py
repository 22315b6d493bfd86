"""OaTrainingSession: a thread-safe control channel for a running training loop
(Source/Public/Oa/Ml/TrainingSession.h:15-190, Source/Private/Oa/Ml/TrainingSession.cpp).

Any thread may enqueue commands (pause, resume, stop, checkpoint, evaluate, set a parameter, re-capture, rebuild); the
training thread applies them only at step boundaries (`TryBeginStep` / `WaitBeginStep` / `Poll`), so a command never
races a step in flight.  Every applied command bumps the session revision; a command that carries an expected revision
is rejected when the session has moved on (optimistic concurrency for UIs).  Registered parameters are classed Hot
(applied at once; device-resident optimizer state makes a learning-rate change replay-safe), Recapture (applied, then the
captured program is dropped and re-captured), Rebuild (handed to the rebuild handler) or Immutable (rejected).
Snapshots and command results are kept in bounded rings.
"""
from __future__ import annotations

import enum
import threading
from collections import deque
from dataclasses import dataclass, field
from typing import Callable, Optional

from ..core.types import OaStatus, OaStatusCode


class OaTrainingState(enum.IntEnum):
    Running = 0
    Paused = 1
    Stopping = 2
    Completed = 3
    Failed = 4


class OaTrainingCommandKind(enum.IntEnum):
    Pause = 0
    Resume = 1
    Stop = 2
    Checkpoint = 3
    Evaluate = 4
    SetParameter = 5
    RequestRecapture = 6
    RequestRebuild = 7


class OaTrainingCommandDisposition(enum.IntEnum):
    Applied = 0
    Rejected = 1


class OaTrainingParameterClass(enum.IntEnum):
    Hot = 0
    Recapture = 1
    Rebuild = 2
    Immutable = 3


class OaTrainingValueKind(enum.IntEnum):
    Empty = 0
    Boolean = 1
    Integer = 2
    Float = 3
    String = 4


@dataclass
class OaTrainingValue:
    Kind: OaTrainingValueKind = OaTrainingValueKind.Empty
    Bool: bool = False
    Integer: int = 0
    Float: float = 0.0
    String: str = ""

    @staticmethod
    def FromBool(v: bool): return OaTrainingValue(OaTrainingValueKind.Boolean, Bool=bool(v))
    @staticmethod
    def FromInteger(v: int): return OaTrainingValue(OaTrainingValueKind.Integer, Integer=int(v))
    @staticmethod
    def FromFloat(v: float): return OaTrainingValue(OaTrainingValueKind.Float, Float=float(v))
    @staticmethod
    def FromString(v: str): return OaTrainingValue(OaTrainingValueKind.String, String=str(v))

    def AsNumber(self) -> Optional[float]:
        if self.Kind == OaTrainingValueKind.Integer:
            return float(self.Integer)
        if self.Kind == OaTrainingValueKind.Float:
            return self.Float
        return None


@dataclass
class OaTrainingCommand:
    Sequence: int = 0
    ExpectedRevision: int = 0
    Kind: OaTrainingCommandKind = OaTrainingCommandKind.Pause
    Parameter: str = ""
    Value: OaTrainingValue = field(default_factory=OaTrainingValue)


@dataclass
class OaTrainingCommandResult:
    Sequence: int = 0
    Revision: int = 0
    Disposition: OaTrainingCommandDisposition = OaTrainingCommandDisposition.Rejected
    State: OaTrainingState = OaTrainingState.Running
    Status: OaStatus = field(default_factory=OaStatus.Ok)


@dataclass
class OaTrainingMetricSample:
    Name: str = ""
    Value: float = 0.0
    Step: int = 0


@dataclass
class OaTrainingSnapshot:
    Revision: int = 0
    State: OaTrainingState = OaTrainingState.Running
    Step: int = 0
    Epoch: int = 0
    LearningRate: float = 0.0
    Loss: float = 0.0
    GpuMs: float = 0.0
    WallMs: float = 0.0
    Metrics: list = field(default_factory=list)


@dataclass
class OaTrainingParameterDesc:
    Name: str = ""
    Class: OaTrainingParameterClass = OaTrainingParameterClass.Hot
    Kind: OaTrainingValueKind = OaTrainingValueKind.Float
    Minimum: Optional[float] = None
    Maximum: Optional[float] = None
    Get: Optional[Callable[[], OaTrainingValue]] = None
    Set: Optional[Callable[[OaTrainingValue], OaStatus]] = None


@dataclass
class OaTrainingSessionHandlers:
    Checkpoint: Optional[Callable[[], OaStatus]] = None
    Evaluate: Optional[Callable[[], OaStatus]] = None
    Rebuild: Optional[Callable[[OaTrainingCommand], OaStatus]] = None


@dataclass
class OaTrainingSessionConfig:
    CommandCapacity: int = 64
    ResultCapacity: int = 128
    SnapshotCapacity: int = 256
    Handlers: OaTrainingSessionHandlers = field(default_factory=OaTrainingSessionHandlers)


class OaTrainingSession:
    def __init__(self, training, config: Optional[OaTrainingSessionConfig] = None):
        self._training = training
        self._cfg = config or OaTrainingSessionConfig()
        self._lock = threading.Lock()
        self._wake = threading.Condition(self._lock)
        self._queue: deque = deque()
        self._results: deque = deque(maxlen=self._cfg.ResultCapacity)
        self._snapshots: deque = deque(maxlen=self._cfg.SnapshotCapacity)
        self._params: dict[str, OaTrainingParameterDesc] = {}
        self._metrics: dict[str, OaTrainingMetricSample] = {}
        self._state = OaTrainingState.Running
        self._revision = 0
        self._next_sequence = 1

    # ---- producers (any thread)
    def Enqueue(self, command: OaTrainingCommand):
        """Returns (sequence, status); the sequence identifies the command's result."""
        with self._wake:
            if self._state in (OaTrainingState.Completed, OaTrainingState.Failed):
                return 0, OaStatus.Error(OaStatusCode.FailedPrecondition, "the training session has ended")
            if len(self._queue) >= self._cfg.CommandCapacity:
                return 0, OaStatus.Error(OaStatusCode.ResourceExhausted, "command queue is full")
            command.Sequence = self._next_sequence
            self._next_sequence += 1
            self._queue.append(command)
            self._wake.notify_all()
            return command.Sequence, OaStatus.Ok()

    def _simple(self, kind, rev, name="", value=None):
        return self.Enqueue(OaTrainingCommand(0, rev, kind, name, value or OaTrainingValue()))

    def Pause(self, expected_revision: int = 0): return self._simple(OaTrainingCommandKind.Pause, expected_revision)
    def Resume(self, expected_revision: int = 0): return self._simple(OaTrainingCommandKind.Resume, expected_revision)
    def Stop(self, expected_revision: int = 0): return self._simple(OaTrainingCommandKind.Stop, expected_revision)
    def Checkpoint(self, expected_revision: int = 0): return self._simple(OaTrainingCommandKind.Checkpoint, expected_revision)
    def Evaluate(self, expected_revision: int = 0): return self._simple(OaTrainingCommandKind.Evaluate, expected_revision)
    def RequestRecapture(self, expected_revision: int = 0): return self._simple(OaTrainingCommandKind.RequestRecapture, expected_revision)

    def SetParameter(self, name: str, value: OaTrainingValue, expected_revision: int = 0):
        return self._simple(OaTrainingCommandKind.SetParameter, expected_revision, name, value)

    def RequestRebuild(self, config: OaTrainingValue, expected_revision: int = 0):
        return self._simple(OaTrainingCommandKind.RequestRebuild, expected_revision, "", config)

    # ---- the training thread
    def RegisterParameter(self, desc: OaTrainingParameterDesc) -> OaStatus:
        with self._lock:
            if not desc.Name or desc.Name in self._params:
                return OaStatus.Error(OaStatusCode.AlreadyExists, f"parameter '{desc.Name}' is empty or already registered")
            self._params[desc.Name] = desc
        return OaStatus.Ok()

    def Parameter(self, name: str) -> Optional[OaTrainingValue]:
        with self._lock:
            d = self._params.get(name)
        return d.Get() if d is not None and d.Get is not None else None

    def Poll(self) -> OaStatus:
        """Applies every queued command (step boundary only)."""
        while True:
            with self._lock:
                if not self._queue:
                    return OaStatus.Ok()
                cmd = self._queue.popleft()
            st = self._apply(cmd)
            with self._wake:
                applied = bool(st)
                if applied:
                    self._revision += 1
                self._results.append(OaTrainingCommandResult(
                    cmd.Sequence, self._revision, OaTrainingCommandDisposition.Applied if applied else OaTrainingCommandDisposition.Rejected,
                    self._state, st))
                self._wake.notify_all()

    def _apply(self, cmd: OaTrainingCommand) -> OaStatus:
        K = OaTrainingCommandKind
        if cmd.ExpectedRevision and cmd.ExpectedRevision != self._revision:
            return OaStatus.Error(OaStatusCode.Aborted, f"expected revision {cmd.ExpectedRevision}, session is at {self._revision}")
        if cmd.Kind == K.Pause:
            if self._state != OaTrainingState.Running:
                return OaStatus.Error(OaStatusCode.FailedPrecondition, "not running")
            self._state = OaTrainingState.Paused
            return OaStatus.Ok()
        if cmd.Kind == K.Resume:
            if self._state != OaTrainingState.Paused:
                return OaStatus.Error(OaStatusCode.FailedPrecondition, "not paused")
            self._state = OaTrainingState.Running
            return OaStatus.Ok()
        if cmd.Kind == K.Stop:
            self._state = OaTrainingState.Stopping
            self._training.RequestStop()
            return OaStatus.Ok()
        if cmd.Kind in (K.Checkpoint, K.Evaluate):
            h = self._cfg.Handlers.Checkpoint if cmd.Kind == K.Checkpoint else self._cfg.Handlers.Evaluate
            return h() if h is not None else OaStatus.Error(OaStatusCode.Unimplemented, "no handler installed")
        if cmd.Kind == K.RequestRecapture:
            self._training.RequestRecapture()
            return OaStatus.Ok()
        if cmd.Kind == K.RequestRebuild:
            h = self._cfg.Handlers.Rebuild
            return h(cmd) if h is not None else OaStatus.Error(OaStatusCode.Unimplemented, "no rebuild handler installed")
        # SetParameter
        d = self._params.get(cmd.Parameter)
        if d is None:
            return OaStatus.Error(OaStatusCode.NotFound, f"unknown parameter '{cmd.Parameter}'")
        if d.Class == OaTrainingParameterClass.Immutable:
            return OaStatus.Error(OaStatusCode.PermissionDenied, f"parameter '{d.Name}' is immutable")
        v = cmd.Value
        num = v.AsNumber()
        kinds_ok = v.Kind == d.Kind or (d.Kind == OaTrainingValueKind.Float and v.Kind == OaTrainingValueKind.Integer)
        if not kinds_ok:
            return OaStatus.Error(OaStatusCode.InvalidArgument, f"parameter '{d.Name}' expects {d.Kind.name}")
        if num is not None and ((d.Minimum is not None and num < d.Minimum) or (d.Maximum is not None and num > d.Maximum)):
            return OaStatus.Error(OaStatusCode.OutOfRange, f"parameter '{d.Name}' = {num} is outside [{d.Minimum}, {d.Maximum}]")
        if d.Class == OaTrainingParameterClass.Rebuild:
            h = self._cfg.Handlers.Rebuild
            return h(cmd) if h is not None else OaStatus.Error(OaStatusCode.Unimplemented, "no rebuild handler installed")
        st = d.Set(v) if d.Set is not None else OaStatus.Error(OaStatusCode.Unimplemented, f"parameter '{d.Name}' has no setter")
        if st and d.Class == OaTrainingParameterClass.Recapture:
            self._training.RequestRecapture()
        return st

    def TryBeginStep(self) -> bool:
        """Applies pending commands; True when the loop may run a step now."""
        self.Poll()
        with self._lock:
            return self._state == OaTrainingState.Running

    def WaitBeginStep(self, poll_seconds: float = 0.05) -> bool:
        """Like TryBeginStep but sleeps while paused; False once the session is stopping or has ended."""
        while True:
            self.Poll()
            with self._wake:
                if self._state == OaTrainingState.Running:
                    return True
                if self._state != OaTrainingState.Paused:
                    return False
                if not self._queue:
                    self._wake.wait(poll_seconds)

    def PublishMetric(self, name: str, value: float) -> None:
        with self._lock:
            self._metrics[name] = OaTrainingMetricSample(name, float(value), self._training.StepCount())

    def OnStepCompleted(self, training=None) -> None:
        t = training or self._training
        with self._lock:
            self._snapshots.append(OaTrainingSnapshot(self._revision, self._state, t.StepCount(), t.Epoch(), float(t.Opt_.Lr()), float(t.LastLoss()),
                                                      t.LastGpuMs(), t.WallMsPerStep(), list(self._metrics.values())))

    def OnReset(self, training=None) -> None:
        with self._lock:
            self._snapshots.clear()
            self._metrics.clear()
            self._state = OaTrainingState.Running

    def OnFinished(self, status: OaStatus, training=None) -> None:
        with self._wake:
            self._state = OaTrainingState.Completed if status else OaTrainingState.Failed
            self._wake.notify_all()

    # ---- observers (any thread)
    def State(self) -> OaTrainingState:
        with self._lock:
            return self._state

    def Revision(self) -> int:
        with self._lock:
            return self._revision

    def LatestSnapshot(self) -> Optional[OaTrainingSnapshot]:
        with self._lock:
            return self._snapshots[-1] if self._snapshots else None

    def ResultsAfter(self, sequence: int) -> list:
        with self._lock:
            return [r for r in self._results if r.Sequence > sequence]

    def TakeResults(self) -> list:
        with self._lock:
            out = list(self._results)
            self._results.clear()
            return out
