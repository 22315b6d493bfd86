"""Learning-rate schedules (Source/Public/Oa/Ml/LrScheduler.h:16-165, Source/Private/Oa/Ml/Callback/LrScheduler.cpp).

A schedule is a pure function of the step index, `GetLr(step)`; `Apply(optimizer)` sets the optimizer's rate for its
current step.  Because the optimizers keep the rate in a device-resident state word, changing it never invalidates a
captured training program.
"""
from __future__ import annotations

import enum
import math
from typing import Optional, Sequence


class OaLRScheduler:
    def GetLr(self, step: int) -> float:
        raise NotImplementedError

    def Apply(self, optimizer) -> None:
        optimizer.SetLr(self.GetLr(int(optimizer.StepCount())))


def _half_cosine(lo: float, hi: float, t: float) -> float:
    """hi at t = 0 falling to lo at t = 1 along half a cosine period."""
    return lo + 0.5 * (hi - lo) * (1.0 + math.cos(math.pi * t))


class OaCosineScheduler(OaLRScheduler):
    def __init__(self, max_lr: float, min_lr: float, total_steps: int):
        self.MaxLr, self.MinLr, self.TotalSteps = float(max_lr), float(min_lr), int(total_steps)

    def GetLr(self, step: int) -> float:
        if step >= self.TotalSteps:
            return self.MinLr
        return _half_cosine(self.MinLr, self.MaxLr, step / self.TotalSteps)


class OaWarmupScheduler(OaLRScheduler):
    """Linear ramp (step + 1) / warmup of the target rate, then `after` (re-based to step 0) or the constant target."""

    def __init__(self, target_lr: float, warmup_steps: int, after: Optional[OaLRScheduler] = None):
        self.TargetLr, self.WarmupSteps, self.After = float(target_lr), int(warmup_steps), after

    def GetLr(self, step: int) -> float:
        if step < self.WarmupSteps:
            return self.TargetLr * (step + 1) / self.WarmupSteps
        return self.After.GetLr(step - self.WarmupSteps) if self.After is not None else self.TargetLr


class OaOneCycleScheduler(OaLRScheduler):
    def __init__(self, max_lr: float, total_steps: int, pct_start: float = 0.3, div_factor: float = 25.0, final_div_factor: float = 1e4):
        self.MaxLr, self.TotalSteps, self.PctStart = float(max_lr), int(total_steps), float(pct_start)
        self.DivFactor, self.FinalDivFactor = float(div_factor), float(final_div_factor)

    def GetLr(self, step: int) -> float:
        floor = self.MaxLr / self.DivFactor / self.FinalDivFactor
        up = self.PctStart * self.TotalSteps
        down = self.TotalSteps - up
        if up > 0 and step <= up:
            return _half_cosine(self.MaxLr, floor, step / up)          # rising: reversed arguments
        if down > 0:
            return _half_cosine(floor, self.MaxLr, min(1.0, (step - up) / down))
        return floor


class OaCyclicMode(enum.IntEnum):
    Triangular = 0
    Triangular2 = 1
    ExpRange = 2


class OaCyclicScheduler(OaLRScheduler):
    def __init__(self, base_lr: float, max_lr: float, step_size_up: int, mode: OaCyclicMode = OaCyclicMode.Triangular, gamma: float = 1.0):
        self.BaseLr, self.MaxLr, self.StepSizeUp, self.Mode, self.Gamma = float(base_lr), float(max_lr), int(step_size_up), mode, float(gamma)

    def GetLr(self, step: int) -> float:
        cycle = math.floor(step / (2.0 * self.StepSizeUp))
        x = abs(step / self.StepSizeUp - 2.0 * cycle - 1.0)
        scale = {OaCyclicMode.Triangular: 1.0, OaCyclicMode.Triangular2: 0.5 ** cycle, OaCyclicMode.ExpRange: self.Gamma ** step}[self.Mode]
        return self.BaseLr + (self.MaxLr - self.BaseLr) * max(0.0, 1.0 - x) * scale


class OaCosineWarmRestartsScheduler(OaLRScheduler):
    def __init__(self, max_lr: float, t0: int, t_mult: int = 1, eta_min: float = 0.0):
        self.MaxLr, self.T0, self.TMult, self.EtaMin = float(max_lr), int(t0), int(t_mult), float(eta_min)

    def GetLr(self, step: int) -> float:
        period, start = self.T0, 0
        if self.TMult == 1:
            start = step - step % self.T0
        else:
            while start + period <= step:
                start += period
                period *= self.TMult
        return _half_cosine(self.EtaMin, self.MaxLr, (step - start) / period)


class OaPlateauMode(enum.IntEnum):
    Min = 0
    Max = 1


class OaReduceOnPlateauScheduler(OaLRScheduler):
    """Stateful: feed `Step(metric)` once per evaluation; the rate drops by `factor` after more than `patience` evaluations
    without an improvement larger than `threshold`."""

    def __init__(self, initial_lr: float, factor: float = 0.1, patience: int = 10, threshold: float = 1e-4, min_lr: float = 0.0,
                 mode: OaPlateauMode = OaPlateauMode.Min):
        self.CurrentLr, self.Factor, self.Patience, self.Threshold = float(initial_lr), float(factor), int(patience), float(threshold)
        self.MinLr, self.Mode = float(min_lr), mode
        self.Best = 1e30 if mode == OaPlateauMode.Min else -1e30
        self.NumBadEpochs = 0

    def Step(self, metric: float) -> None:
        better = metric < self.Best - self.Threshold if self.Mode == OaPlateauMode.Min else metric > self.Best + self.Threshold
        if better:
            self.Best, self.NumBadEpochs = float(metric), 0
        else:
            self.NumBadEpochs += 1
        if self.NumBadEpochs > self.Patience:
            self.CurrentLr = max(self.CurrentLr * self.Factor, self.MinLr)
            self.NumBadEpochs = 0

    def GetLr(self, step: int) -> float:
        return self.CurrentLr


class OaSequentialScheduler(OaLRScheduler):
    """Schedule i runs from milestone i-1 (re-based to its own step 0) to milestone i; the last one runs to the end."""

    def __init__(self, schedulers: Sequence[OaLRScheduler], milestones: Sequence[int]):
        self.Schedulers, self.Milestones = list(schedulers), [int(m) for m in milestones]

    def GetLr(self, step: int) -> float:
        if not self.Schedulers:
            return 0.0
        offset = 0
        for sched, stone in zip(self.Schedulers, self.Milestones):
            if step < stone:
                return sched.GetLr(step - offset)
            offset = stone
        return self.Schedulers[-1].GetLr(step - offset)


class OaLinearWarmupCosineScheduler(OaLRScheduler):
    """Linear warm-up to max_lr, then cosine decay to min_lr; indexed by the 1-based optimizer step (steps 0 and 1 agree)."""

    def __init__(self, warmup_steps: int, total_steps: int, max_lr: float, min_lr: float):
        w = max(0, int(warmup_steps))
        span = max(1, int(total_steps) - int(warmup_steps))
        self.Inner = OaWarmupScheduler(max_lr, w, OaCosineScheduler(max_lr, min_lr, span))

    def GetLr(self, step: int) -> float:
        return self.Inner.GetLr(max(0, step - 1))
