"""Training callbacks (Source/Public/Oa/Ml/Callbacks.h:49-760): progress bar, validation, checkpointing, early stopping,
learning-rate scheduling, CSV logging, end-of-run summary and phase schedules.  Hooks receive the OaItTraining iterator;
a hook that returns a failed OaStatus stops the run.
"""
from __future__ import annotations

import enum
import sys
import time
from dataclasses import dataclass, field
from typing import Callable, Optional

from ..core.types import OaStatus
from .checkpoint import OaCheckpointManager
from .metric import OaMetric, OaMetricLoss
from .training import OaCallback


class OaCbProgressBar(OaCallback):
    """One line per epoch (or per run), redrawn in place: [####......] step/total loss=... it/s."""

    def __init__(self, bar_width: int = 10, stream=None):
        self.BarWidth, self._out, self._t0 = int(bar_width), stream or sys.stdout, 0.0

    def OnTrainBegin(self, training):
        self._t0 = time.perf_counter()

    def OnStepEnd(self, training, step, loss):
        spe = training.Config.StepsPerEpoch
        total = spe if spe > 0 else training.Config.TotalSteps
        done = (step % spe or spe) if spe > 0 else step
        fill = int(self.BarWidth * done / max(1, total))
        rate = step / max(1e-9, time.perf_counter() - self._t0)
        self._out.write(f"\r[{'#' * fill}{'.' * (self.BarWidth - fill)}] {done}/{total} loss={loss:.4f} {rate:.1f} it/s")
        self._out.flush()

    def OnEpochEnd(self, training, epoch):
        self._out.write(f"  epoch {epoch + 1} mean loss {training.EpochMeanLoss():.4f}\n")

    def OnTrainEnd(self, training):
        self._out.write("\n")
        self._out.flush()


@dataclass
class OaValidationResult:
    Loss: float = 0.0
    Accuracy: float = 0.0
    Samples: int = 0
    Extra: dict = field(default_factory=dict)


class OaCbValidation(OaCallback):
    """Runs `eval_fn(training) -> OaValidationResult` at every epoch end, or every `step_interval` steps when the run has
    no epochs (and once more at the end if the last step was not evaluated)."""

    def __init__(self, eval_fn: Callable, metric_name: str = "val_loss", step_interval: int = 0):
        self.Eval, self.Metric_, self.StepInterval = eval_fn, OaMetricLoss(metric_name), int(step_interval)
        self.LastResult_, self.LastSeconds_, self._last_eval_step = OaValidationResult(), 0.0, -1

    def _run(self, training):
        t0 = time.perf_counter()
        self.LastResult_ = self.Eval(training)
        self.LastSeconds_ = time.perf_counter() - t0
        self._last_eval_step = training.StepCount()
        self.Metric_.Reset()
        self.Metric_.Update(float(self.LastResult_.Loss), max(1, int(self.LastResult_.Samples)))

    def OnStepEnd(self, training, step, loss):
        if not training.HasEpochs() and self.StepInterval > 0 and step % self.StepInterval == 0:
            self._run(training)

    def OnEpochEnd(self, training, epoch):
        if training.HasEpochs():
            self._run(training)

    def OnTrainEnd(self, training):
        if not training.HasEpochs() and self._last_eval_step != training.StepCount():
            self._run(training)

    def MetricPtr(self) -> OaMetricLoss:
        return self.Metric_

    Metric = MetricPtr

    def LastResult(self) -> OaValidationResult:
        return self.LastResult_

    def LastSeconds(self) -> float:
        return self.LastSeconds_


class OaCbCheckpoint(OaCallback):
    """Resumable snapshot every `save_every` steps (never on an epoch boundary), best-model file at every epoch end when
    the metric (given metric, else the epoch mean loss) improved, and optionally the best weights restored at the end."""

    def __init__(self, manager: OaCheckpointManager, model, optimizer, save_every: int = 0, metric: Optional[OaMetric] = None,
                 restore_best: bool = True, verbose: bool = True):
        self.Mgr, self.Model, self.Opt, self.SaveEvery = manager, model, optimizer, int(save_every)
        self.Metric, self.RestoreBest, self.Verbose = metric, restore_best, verbose
        self.Status = OaStatus.Ok()
        self._saved_best = False

    def GetStatus(self) -> OaStatus:
        return self.Status

    def _metric(self, training) -> float:
        value = float(self.Metric.Value()) if self.Metric is not None else float(training.EpochMeanLoss())
        return OaCheckpointManager._agreed(self.Opt, value)      # the same number on every rank

    def OnStepEnd(self, training, step, loss):
        if not self.Status or self.SaveEvery <= 0 or training.IsEpochBoundary() or step % self.SaveEvery:
            return None
        if self.Verbose:
            print(f"\nStep {step}: loss = {loss:.6f} - saving resumable checkpoint", flush=True)
        self.Status = self.Mgr.SaveIncremental(self.Model, self.Opt, step, float(loss), "loss")   # agrees on the loss itself
        return self.Status

    def OnEpochEnd(self, training, epoch):
        if not self.Status:
            return self.Status
        metric = self._metric(training)
        if self.Mgr.IsBetter(metric):
            if self.Verbose:
                print(f"\nEpoch {epoch + 1}: {self.Mgr.MetricName()} improved {self.Mgr.GetBestMetric():.6f} -> {metric:.6f}, saving best", flush=True)
            self.Status = self.Mgr.MaybeSave(self.Model, self.Opt, training.StepCount(), metric, agreed=True)
            self._saved_best = bool(self.Status)
        return self.Status

    def OnTrainEnd(self, training):
        if self.Status and self.RestoreBest and self._saved_best:
            self.Status = self.Mgr.LoadBestInto(self.Model, self.Opt)
        return self.Status


class OaEarlyStopMode(enum.IntEnum):
    Min = 0
    Max = 1


class OaCbEarlyStop(OaCallback):
    def __init__(self, patience: int = 5, min_delta: float = 1e-4, mode: OaEarlyStopMode = OaEarlyStopMode.Min,
                 metric: Optional[OaMetric] = None):
        self.Patience, self.MinDelta, self.Mode, self.Metric = int(patience), float(min_delta), mode, metric
        self.BestMetric = float("inf") if mode == OaEarlyStopMode.Min else float("-inf")
        self.BadEpochs, self._stop = 0, False

    def OnEpochEnd(self, training, epoch):
        value = float(self.Metric.Value()) if self.Metric is not None else float(training.EpochMeanLoss())
        better = value < self.BestMetric - self.MinDelta if self.Mode == OaEarlyStopMode.Min else value > self.BestMetric + self.MinDelta
        if better:
            self.BestMetric, self.BadEpochs = value, 0
            return
        self.BadEpochs += 1
        if self.BadEpochs >= self.Patience:
            print(f"Epoch {epoch + 1}: early stopping - no improvement for {self.BadEpochs} epochs (best {self.BestMetric:.6f})")
            self._stop = True
            training.RequestStop()

    def ShouldStop(self) -> bool:
        return self._stop


class OaCbLrScheduler(OaCallback):
    """After step n the rate for step n + 1 is installed (schedules are indexed by the 1-based step)."""

    def __init__(self, scheduler, optimizer):
        self.Scheduler, self.Opt = scheduler, optimizer

    def OnStepEnd(self, training, step, loss):
        self.Opt.SetLr(self.Scheduler.GetLr(step + 1))


class OaCbCsvLogger(OaCallback):
    HEADER = ("epoch,step,batch_size,sequence_length,sequence_unit,source_unit,loss,gpu_ms,wall_ms_per_step,wall_samples_per_second,"
              "gpu_samples_per_second,wall_units_per_second,gpu_units_per_second,wall_source_units_per_second,"
              "gpu_source_units_per_second\n")

    def __init__(self, path: str):
        self.Path, self._f = path, None

    def OnTrainBegin(self, training):
        self._f = open(self.Path, "w")
        self._f.write(self.HEADER)
        self._f.flush()

    def OnStepEnd(self, training, step, loss):
        if self._f is None:
            return
        c = training.Config
        self._f.write(f"{training.Epoch()},{step},{c.BatchSize},{c.SequenceLength},{c.SequenceUnit},{c.SourceUnit},{loss},"
                      f"{training.LastGpuMs()},{training.WallMsPerStep()},{training.WallSamplesPerSecond()},{training.GpuSamplesPerSecond()},"
                      f"{training.WallUnitsPerSecond()},{training.GpuUnitsPerSecond()},{training.WallSourceUnitsPerSecond()},"
                      f"{training.GpuSourceUnitsPerSecond()}\n")

    def OnEpochEnd(self, training, epoch):
        if self._f is not None:
            self._f.flush()

    def OnTrainEnd(self, training):
        if self._f is not None:
            self._f.close()
            self._f = None


class OaCbSummary(OaCallback):
    """Prints first / final loss, step count, device and wall time per step and throughput when training ends."""

    def __init__(self, track_initial_loss: bool = True, stream=None):
        self.TrackInitial, self.InitialLoss, self._out = track_initial_loss, None, stream or sys.stdout

    def OnStepEnd(self, training, step, loss):
        if self.TrackInitial and self.InitialLoss is None:
            self.InitialLoss = float(loss)

    def OnTrainEnd(self, training):
        st = training.GpuTimingStats()
        first = f"{self.InitialLoss:.4f} -> " if self.InitialLoss is not None else ""
        self._out.write(f"steps {training.StepCount()}  loss {first}{training.LastLoss():.4f}  device ms/step mean {st.MeanMs:.3f} "
                        f"p50 {st.P50Ms:.3f} p95 {st.P95Ms:.3f}  wall ms/step {training.WallMsPerStep():.3f}  "
                        f"{training.WallUnitsPerSecond():.0f} {training.Config.SequenceUnit}/s\n")


class OaCbPhase(OaCallback):
    """A named sequence of phases, each a number of epochs; `on_phase_begin(index, phase)` fires when a phase starts."""

    @dataclass
    class Phase:
        Id: str
        Epochs: int = 0
        Steps: int = 0

    def __init__(self):
        self.Phases: list = []
        self.OnPhaseBegin: Optional[Callable] = None
        self._current = -1

    def AddPhase(self, ident: str, epochs: int, steps: int) -> None:
        self.Phases.append(OaCbPhase.Phase(ident, int(epochs), int(steps)))

    def SetOnPhaseBegin(self, fn: Callable) -> None:
        self.OnPhaseBegin = fn

    def CurrentPhase(self) -> int:
        return self._current

    def OnEpochBegin(self, training, epoch):
        if not self.Phases:
            return
        before, idx = 0, len(self.Phases) - 1
        for i, ph in enumerate(self.Phases):
            if epoch < before + ph.Epochs:
                idx = i
                break
            before += ph.Epochs
        if idx != self._current:
            self._current = idx
            ph = self.Phases[idx]
            print(f"\nPhase {idx + 1}/{len(self.Phases)} - {ph.Id}: {ph.Epochs} epochs, {ph.Steps} steps")
            if self.OnPhaseBegin is not None:
                self.OnPhaseBegin(idx, ph)
