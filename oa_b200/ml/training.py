"""Training loop objects: OaItTraining, OaTrainingProgram (CUDA-graph capture / replay), timing stats.

Reference: Source/Public/Oa/Ml/ItTraining.h:58-387 and ItTraining.cpp:245-553 (iterator-style step life cycle,
exact per-step sync, loss readback, GPU timer statistics, throughput in samples / units / source units, callbacks),
Source/Public/Oa/Ml/TrainingProgram.h:21-179 and TrainingProgram.cpp:255-448 (capture of a recorded step and
replay).  Where the reference copies graph nodes into a compiled Vulkan graph, the step is captured here into a
CUDA graph: step 1 runs eagerly (it creates lazy optimizer state and scratch buffers), the next step is captured,
every later step only refills the static input buffers and replays.  Mutable scalars (optimizer step, learning
rate) live in device memory, RNG offsets are advanced by the captured kernels' arguments being fixed per replay
only for ops that are replay-safe; dropout inside a captured program is rejected like the reference rejects raw
Philox nodes.
"""
from __future__ import annotations

import os
import contextlib
import time
from dataclasses import dataclass, field
from typing import Callable, Optional

import torch

from ..core.matrix import OaMatrix
from ..core.types import OaStatus, OaStatusCode
from ..runtime import engine as RT
from ..utils import envflag


@dataclass
class OaItTrainingConfig:
    TotalSteps: int = 100
    BatchSize: int = 1
    SequenceLength: int = 1
    SequenceUnit: str = "token"
    SourceUnit: str = "byte"
    TimerName: str = "train"
    StepsPerEpoch: int = 0
    Program: bool = False            # capture the step into a CUDA graph from step 2 on
    ValidateEvery: int = 0           # with a program: every N steps run the step eagerly, compare its node structure with
                                     # the captured one and drop the program when it changed (0: only on request)
    SyncEveryStep: bool = True       # exact per-step loss readback (the reference always does)
    LogEvery: int = 0


@dataclass
class OaGpuTimingStats:
    Count: int = 0
    MeanMs: float = 0.0
    MinMs: float = 0.0
    P50Ms: float = 0.0
    P95Ms: float = 0.0


@dataclass
class OaTrainingPhaseStats:
    BodyMs: float = 0.0
    OptimizerMs: float = 0.0
    CaptureMs: float = 0.0
    SubmitMs: float = 0.0
    WaitMs: float = 0.0
    ScalarMs: float = 0.0
    CallbackMs: float = 0.0


class OaTrainingProgram:
    """A captured training step.  `Capture(fn)` records everything `fn` launches into a CUDA graph and keeps the tensors it
    returns alive as static outputs; `Replay()` launches the graph, `Wait()` blocks until it finished.

    Stages of a capture (`StageLog` lists the ones that ran, with their milliseconds):
      collect      `fn` runs under stream capture while the context collects its nodes and the marks of ops that freeze
                   host values into their launches;
      rng-rewrite  random ops inside `fn` read (seed, base offset) from device memory and the step is closed by a launch
                   that advances the base by the counters the step consumed, so every replay draws fresh numbers, the
                   same ones the eager step would have drawn;
      validate     replay-unsafe marks refuse the capture; the collected nodes go through the native compute graph
                   (hazards, levels) and their structure hash is stored;
      instantiate  the CUDA graph is instantiated (by the end of the capture);
      ready.
    `Verify(nodes)` compares the structure hash of a freshly recorded step with the captured one: OaItTraining re-records
    a step eagerly every `ValidateEvery` steps and drops a program whose step has changed shape instead of replaying it."""

    Stages = ("collect", "rng-rewrite", "validate", "instantiate", "ready")

    def __init__(self):
        self._graph: Optional[torch.cuda.CUDAGraph] = None
        self._outputs = None
        self._event = None
        self.CaptureMs = 0.0
        self.NodeCount = 0
        self.Replays = 0
        self.StageLog: list = []
        self.StructureHash = 0
        self.GraphHash = 0
        self.Levels = 0
        self.Barriers = 0
        self.RngCountersPerStep = 0
        self.Unsafe: list = []

    def IsCaptured(self) -> bool:
        return self._graph is not None

    def Capture(self, fn: Callable[[], object]) -> OaStatus:
        from ..core import fn_matrix as F
        eng = RT.get_engine()
        if not eng.IsCuda():
            return OaStatus.Error(OaStatusCode.FailedPrecondition, "program capture needs a CUDA engine")
        ctx = RT.OaContext.GetDefault()
        t0 = time.perf_counter()
        torch.cuda.synchronize()
        n0 = ctx.NodeCount()
        g = torch.cuda.CUDAGraph()
        self.StageLog = []
        F.BeginProgramRng()
        ctx.BeginCollect()
        try:
            # thread-local capture mode: a communication watchdog thread may query events while we capture
            with torch.cuda.graph(g, capture_error_mode="thread_local"):
                self._outputs = fn()
                self.RngCountersPerStep = F.EndProgramRng()
        except Exception as e:  # leave no half-captured graph behind
            F.EndProgramRng()
            ctx.EndCollect()
            self._graph = None
            return OaStatus.Error(OaStatusCode.Internal, f"capture failed: {e}")
        t1 = time.perf_counter()
        self.StageLog.append(("collect", (t1 - t0) * 1e3))
        if self.RngCountersPerStep:
            self.StageLog.append(("rng-rewrite", 0.0))
        nodes, self.Unsafe = ctx.EndCollect()
        if self.Unsafe:
            self._outputs = None
            return OaStatus.Error(OaStatusCode.FailedPrecondition,
                                  "the step cannot be replayed: " + "; ".join(sorted(set(self.Unsafe))))
        graph, self.StructureHash = RT.OaContext.Compile(nodes)
        self.GraphHash, self.Levels, self.Barriers = graph.Hash(), graph.NumLevels(), graph.NumBarriers()
        self.NodeCount = ctx.NodeCount() - n0
        t2 = time.perf_counter()
        self.StageLog.append(("validate", (t2 - t1) * 1e3))
        self._graph = g
        self.CaptureMs = (time.perf_counter() - t0) * 1e3
        self.StageLog += [("instantiate", 0.0), ("ready", self.CaptureMs)]
        return OaStatus.Ok()

    def Verify(self, nodes) -> OaStatus:
        """Does a freshly recorded step still have the structure that was captured?"""
        _, h = RT.OaContext.Compile(nodes)
        if h != self.StructureHash or len(nodes) != self.NodeCount:
            return OaStatus.Error(OaStatusCode.FailedPrecondition,
                                  f"the recorded step changed ({len(nodes)} nodes, hash {h:016x}) since it was captured "
                                  f"({self.NodeCount} nodes, hash {self.StructureHash:016x})")
        return OaStatus.Ok()

    def Outputs(self):
        return self._outputs

    def Replay(self) -> None:
        from ..core import fn_matrix as F
        self._graph.replay()
        if self.RngCountersPerStep:
            F.AdvanceHostRng(self.RngCountersPerStep)
        self.Replays += 1

    def Wait(self) -> OaStatus:
        return RT.OaContext.GetDefault().Sync()

    def DebugReport(self) -> dict:
        return {"captured": self.IsCaptured(), "nodes": self.NodeCount, "capture_ms": self.CaptureMs, "replays": self.Replays,
                "stages": [s for s, _ in self.StageLog], "structure_hash": f"{self.StructureHash:016x}",
                "graph_hash": f"{self.GraphHash:016x}", "levels": self.Levels, "barriers": self.Barriers,
                "rng_counters_per_step": self.RngCountersPerStep}


class OaAccumulatedStep:
    """A training step made of `accum` micro-steps (forward + backward of one micro-batch into the gradient arenas) and
    one optimizer step, with the MICRO-step captured as a CUDA graph and replayed: the form a tensor-parallel or large
    model trains in, where one step is tens of thousands of launches.

    The first call runs eagerly.  The capture is taken on a micro-step that is not the first of its step: by then every
    gradient buffer has been written once, so each weight-gradient kernel is recorded in its accumulating form, and a
    replay right after ZeroGrad adds to zeros.  `after_backward` (gradient synchronisation of replicated parameters) and
    the optimizers stay outside the graph: they run once per step.  A micro-step that cannot be captured (an operation
    that reads a device value on the host, a host-stepped optimizer inside it) keeps running eagerly and `LastStatus`
    says why.  Fused multi-GPU kernels replay like any other: their epochs and counters live in device memory."""

    def __init__(self, optimizers, micro_step: Callable[[], object], accum: int, after_backward: Optional[Callable[[], None]] = None,
                 program: bool = True):
        self.Optimizers = list(optimizers)
        self.MicroStep = micro_step
        self.Accum = int(accum)
        self.AfterBackward = after_backward or (lambda: None)
        self.UseProgram = bool(program) and RT.get_engine().IsCuda()
        self._program: Optional[OaTrainingProgram] = None
        self._steps = 0
        self.LastStatus = OaStatus.Ok()
        self.Loss = None

    def Program(self) -> Optional[OaTrainingProgram]:
        return self._program

    def IsReplaying(self) -> bool:
        return self._program is not None and self._program.IsCaptured()

    def _capture(self):
        prog = OaTrainingProgram()
        st = prog.Capture(self.MicroStep)
        self.LastStatus = st
        if st.IsOk():
            self._program = prog
            prog.Replay()                    # the capture recorded the micro-step without running it
            return prog.Outputs()
        self.UseProgram = False
        return self.MicroStep()

    def Run(self, feed: Optional[Callable[[], None]] = None):
        """One step: ZeroGrad, `accum` micro-steps (each after `feed()`, which loads the next micro-batch into the static
        input buffers), `after_backward`, every optimizer's Step.  Returns the loss matrix of the last micro-step."""
        for o in self.Optimizers:
            o.ZeroGrad()
        loss = None
        for m in range(self.Accum):
            if feed is not None:
                feed()
            if self.IsReplaying():
                self._program.Replay()
                loss = self._program.Outputs()
            elif self.UseProgram and self._steps >= 1 and (m >= 1 or self.Accum == 1):
                loss = self._capture()
            else:
                loss = self.MicroStep()
        self.AfterBackward()
        for o in self.Optimizers:
            o.Step()
        self._steps += 1
        self.Loss = loss
        return loss


class OaCallback:
    """Hooks fired by OaItTraining (Source/Public/Oa/Ml/Callbacks.h:49-236). Return an OaStatus or None."""

    def OnTrainBegin(self, training): return None
    def OnTrainEnd(self, training): return None
    def OnEpochBegin(self, training, epoch: int): return None
    def OnEpochEnd(self, training, epoch: int): return None
    def OnStepEnd(self, training, step: int, loss: float): return None


OaCbTraining = OaCallback


class OaItTraining:
    def __init__(self, optimizer, config: Optional[OaItTrainingConfig] = None):
        self.Opt_ = optimizer
        self.Config = config or OaItTrainingConfig()
        self._index = 0
        self._started = False
        self._finished = False
        self._stop = False
        self._last_loss = float("nan")
        self._losses: list[float] = []
        self._gpu_ms: list[float] = []
        self._wall0 = 0.0
        self._wall_total = 0.0
        self._step_wall0 = 0.0
        self._source_units = 0
        self._source_units_total = 0
        self._callbacks: list[OaCallback] = []
        self._metrics: list = []
        self._timer = RT.OaGpuTimer(self.Config.TimerName)
        self._program: Optional[OaTrainingProgram] = OaTrainingProgram() if (self.Config.Program or envflag.IsSet("OA_TRAINING_PROGRAM")) else None
        self._static_loss: Optional[OaMatrix] = None
        self.LastStatus = OaStatus.Ok()
        self.Phase = OaTrainingPhaseStats()
        self._epoch = 0
        self._log_phases = envflag.IsSet("OA_LOG_TRAINING_PHASES")

    # ---- configuration
    def AddCallback(self, cb: OaCallback) -> None:
        self._callbacks.append(cb)

    def AddMetric(self, metric) -> None:
        self._metrics.append(metric)

    def Program(self) -> Optional[OaTrainingProgram]:
        return self._program

    # ---- life cycle
    def IsDone(self) -> bool:
        if self._finished or self._stop or self._index >= self.Config.TotalSteps:
            return True
        if not self._started:
            self._started = True
            self._wall0 = time.perf_counter()
            self._fire("OnTrainBegin")
            self._fire("OnEpochBegin", self._epoch)
        self._step_wall0 = time.perf_counter()
        self._timer.Begin()
        return False

    def RequestStop(self) -> None:
        self._stop = True

    def StopRequested(self) -> bool:
        return self._stop

    def TotalSteps(self) -> int:
        return self.Config.TotalSteps

    def IsValid(self) -> bool:
        return bool(self.LastStatus)

    def RequestRecapture(self) -> None:
        """Drops the captured program; the next step runs eagerly and the one after captures again."""
        if self._program is not None:
            self._program = OaTrainingProgram()
            self._static_loss = None
            self._recapture_at = self._index + 1

    def Index(self) -> int:
        """Number of completed steps."""
        return self._index

    def RecordSourceUnits(self, n: int) -> None:
        self._source_units = int(n)

    def Step(self, prepare: Optional[Callable[[], None]], record: Callable[[], OaMatrix]) -> float:
        """One step in two phases: `prepare` refills the (static) input buffers, `record` launches zero-grad, forward,
        loss and backward and returns the loss.  With a program configured, `record` + the optimizer step are captured
        at step 2 and replayed afterwards; only `prepare` runs on the host on replay steps."""
        monitor = getattr(self, "_rank_monitor", None)
        if monitor is not None:                      # between steps: nothing of this rank is in flight yet
            monitor.Beat(self._index)
            st = monitor.Check()
            if not st:
                self.LastStatus = st
                self._stop = True
                return float("nan")
        if self._program is not None and self._program.IsCaptured() and (
                getattr(self, "_verify_next", False)
                or (self.Config.ValidateEvery > 0 and self._index > 0 and self._index % self.Config.ValidateEvery == 0)):
            return self._verified_eager_step(prepare, record)
        if self._program is not None and self._program.IsCaptured():
            if prepare is not None:
                prepare()
            t0 = time.perf_counter()
            with self._range("step.replay"):
                self._program.Replay()
            self.Opt_.NotifyProgramReplay()
            self.Phase.SubmitMs = (time.perf_counter() - t0) * 1e3
            return self._finish_step(self._static_loss, stepped=True)
        if prepare is not None:
            prepare()
        if self._program is not None and self._index >= max(1, getattr(self, "_recapture_at", 1)):
            def body():
                loss = record()
                self.Opt_.Step()
                return loss
            st = self._program.Capture(body)
            if not st:
                self.LastStatus = st
                self._stop = True
                return float("nan")
            self.Opt_.Step_ -= 1                    # the capture pass itself did not execute a step
            self._static_loss = self._program.Outputs()
            self._program.Replay()
            self.Opt_.NotifyProgramReplay()
            return self._finish_step(self._static_loss, stepped=True)
        t0 = time.perf_counter()
        with self._range("step.body"):
            loss = record()
        self.Phase.BodyMs = (time.perf_counter() - t0) * 1e3
        return self.Next(loss)

    def RequestVerify(self) -> None:
        """The next step runs eagerly and its recorded structure is compared with the captured program."""
        self._verify_next = True

    def _verified_eager_step(self, prepare, record) -> float:
        """One eager step whose node sequence is checked against the captured program.  The step does the real work of
        this iteration; on a mismatch the program is dropped (the following steps re-capture) and the status says why."""
        self._verify_next = False
        if prepare is not None:
            prepare()
        ctx = RT.OaContext.GetDefault()
        ctx.BeginCollect()
        loss = record()
        self.Opt_.Step()
        nodes, _ = ctx.EndCollect()
        st = self._program.Verify(nodes)
        self.LastVerify = st
        if not st:
            self.RequestRecapture()
        return self._finish_step(loss, stepped=True)

    def SetRankMonitor(self, monitor) -> None:
        """Check the peers' heartbeats before every `Step`: a rank that failed or fell silent stops this loop with an
        `Unavailable` status before the next launch (see `oa_b200.parallel.health.OaRankMonitor`)."""
        self._rank_monitor = monitor

    def _range(self, name: str):
        """Profiler range around a phase of the step when OA_NVTX is set (a system profiler then shows the phases)."""
        if not envflag.IsSet("OA_NVTX"):
            return contextlib.nullcontext()
        from ..utils.perf import OaNvtxRange
        return OaNvtxRange(name)

    def Next(self, loss: OaMatrix) -> float:
        t0 = time.perf_counter()
        with self._range("step.optimizer"):
            self.Opt_.Step()
        self.Phase.OptimizerMs = (time.perf_counter() - t0) * 1e3
        return self._finish_step(loss, stepped=True)

    def _finish_step(self, loss: OaMatrix, stepped: bool) -> float:
        ctx = RT.OaContext.GetDefault()
        t0 = time.perf_counter()
        ev = ctx.Submit(self._timer)
        t1 = time.perf_counter()
        if self.Config.SyncEveryStep:
            st = ctx.Wait(ev)
            if not st:
                self.LastStatus = st
                self._stop = True
            t2 = time.perf_counter()
            self._last_loss = loss.Item()
            self._gpu_ms.append(self._timer.ReadbackMs())
            self.Phase.WaitMs = (t2 - t1) * 1e3
            self.Phase.ScalarMs = (time.perf_counter() - t2) * 1e3
        self.Phase.SubmitMs += (t1 - t0) * 1e3
        self._losses.append(self._last_loss)
        self._index += 1
        self._source_units_total += self._source_units
        self._wall_total = time.perf_counter() - self._wall0
        for m in self._metrics:
            if getattr(m, "Name", "") == "loss":
                m.Update(self._last_loss)
        tcb = time.perf_counter()
        self._fire("OnStepEnd", self._index, self._last_loss)
        spe = self.Config.StepsPerEpoch
        if spe and self._index % spe == 0:
            self._fire("OnEpochEnd", self._epoch)
            self._epoch += 1
            if self._index < self.Config.TotalSteps:
                self._fire("OnEpochBegin", self._epoch)
        self.Phase.CallbackMs = (time.perf_counter() - tcb) * 1e3
        if self._log_phases:
            p = self.Phase
            print(f"[oa phases] step {self._index}: body {p.BodyMs:.3f} opt {p.OptimizerMs:.3f} submit {p.SubmitMs:.3f} "
                  f"wait {p.WaitMs:.3f} scalar {p.ScalarMs:.3f} cb {p.CallbackMs:.3f} ms")
        return self._last_loss

    def Finish(self) -> None:
        if self._finished:
            return
        self._finished = True
        ctx = RT.OaContext.GetDefault()
        ctx.Execute()
        ctx.Sync()
        if self._started:
            if not self.Config.StepsPerEpoch:
                self._fire("OnEpochEnd", self._epoch)
            self._fire("OnTrainEnd")
        report = envflag.GetString("OA_GRAPH_REPORT", "")
        if report and report != "1":
            import json
            with open(report, "w") as f:
                json.dump({"nodes": [n[0] for n in ctx.LastGraph()], "program": self._program.DebugReport() if self._program else None}, f)

    def _fire(self, hook: str, *args) -> None:
        for cb in self._callbacks:
            st = getattr(cb, hook)(self, *args)
            if isinstance(st, OaStatus) and not st:
                self.LastStatus = st
                self._stop = True

    # ---- results
    def LastLoss(self) -> float:
        return self._last_loss

    def StepCount(self) -> int:
        return self._index

    def Cfg(self) -> OaItTrainingConfig:
        return self.Config

    def HasEpochs(self) -> bool:
        return self.Config.StepsPerEpoch > 0

    def IsEpochBoundary(self) -> bool:
        spe = self.Config.StepsPerEpoch
        return spe > 0 and self._index > 0 and self._index % spe == 0

    def EpochMeanLoss(self) -> float:
        """Mean loss of the steps of the epoch that is running (or has just ended)."""
        spe = self.Config.StepsPerEpoch
        if not self._losses:
            return float("nan")
        if spe <= 0:
            xs = self._losses
        else:
            done = self._index % spe or spe
            xs = self._losses[-done:]
        return sum(xs) / len(xs)

    def LastGpuMs(self) -> float:
        return self._gpu_ms[-1] if self._gpu_ms else 0.0

    def GpuSamplesPerSecond(self) -> float:
        ms = self.GpuMsPerStep()
        return self.Config.BatchSize / (ms / 1e3) if ms > 0 else 0.0

    def GpuSourceUnitsPerSecond(self) -> float:
        ms = sum(self._gpu_ms)
        return self._source_units_total / (ms / 1e3) if ms > 0 else 0.0

    def Losses(self) -> list:
        return list(self._losses)

    def Epoch(self) -> int:
        return self._epoch

    def GpuTimingStats(self) -> OaGpuTimingStats:
        xs = sorted(self._gpu_ms)
        if not xs:
            return OaGpuTimingStats()
        n = len(xs)
        return OaGpuTimingStats(n, sum(xs) / n, xs[0], xs[n // 2], xs[min(n - 1, int(0.95 * n))])

    def WallMsPerStep(self) -> float:
        return self._wall_total * 1e3 / max(1, self._index)

    def GpuMsPerStep(self) -> float:
        return self.GpuTimingStats().MeanMs

    def WallSamplesPerSecond(self) -> float:
        return self.Config.BatchSize * self._index / max(self._wall_total, 1e-12)

    def WallUnitsPerSecond(self) -> float:
        return self.WallSamplesPerSecond() * self.Config.SequenceLength

    def WallSourceUnitsPerSecond(self) -> float:
        return self._source_units_total / max(self._wall_total, 1e-12)

    def GpuUnitsPerSecond(self) -> float:
        ms = self.GpuMsPerStep()
        return self.Config.BatchSize * self.Config.SequenceLength / (ms / 1e3) if ms > 0 else 0.0
