"""OaCheckpointManager: best-model and rotating incremental checkpoints (Source/Public/Oa/Ml/Checkpoint.h:27-82,
Source/Private/Oa/Ml/Checkpoint.cpp:96-260).

Layout under <Dir>/<ModelName>/:  <ModelName>.oam is the best model so far (weights + optimizer + progress);
checkpoint[_<Context>]/<ModelName>[_<Context>]_step<N>_<metric><value>.oam are resumable snapshots, of which the newest
MaxKeep are kept.  Every file is written by OaModule.Save (temporary file + fsync + rename).
"""
from __future__ import annotations

import os
import re
from dataclasses import dataclass
from typing import Optional

from ..core.types import OaStatus, OaStatusCode
from ..io.oam import OamModel, OamProgress


@dataclass
class OaCheckpointManagerConfig:
    Dir: str = "var/model/dev"
    ModelName: str = "OaModule"
    Context: str = ""
    MaxKeep: int = 5
    SaveBest: bool = True
    MetricName: str = "loss"
    LowerIsBetter: bool = True


class OaCheckpointManager:
    def __init__(self, config: Optional[OaCheckpointManagerConfig] = None):
        self.Config = config or OaCheckpointManagerConfig()
        self.BestMetric = float("inf") if self.Config.LowerIsBetter else float("-inf")
        self._saved: list[tuple[str, float, int]] = []       # (path, metric, step)

    # ---- paths
    def GetModelDir(self) -> str:
        return os.path.join(self.Config.Dir, self.Config.ModelName)

    def GetIncrementalDir(self) -> str:
        return os.path.join(self.GetModelDir(), "checkpoint" + (f"_{self.Config.Context}" if self.Config.Context else ""))

    def GetMasterPath(self) -> str:
        return os.path.join(self.GetModelDir(), self.Config.ModelName + ".oam")

    def BuildFilename(self, step: int, metric: float, metric_name: str = "") -> str:
        ctx = f"_{self.Config.Context}" if self.Config.Context else ""
        return f"{self.Config.ModelName}{ctx}_step{int(step)}_{metric_name or self.Config.MetricName}{metric:.2f}.oam"

    def IsBetter(self, metric: float) -> bool:
        return metric < self.BestMetric if self.Config.LowerIsBetter else metric > self.BestMetric

    def GetBestMetric(self) -> float:
        return self.BestMetric

    def MetricName(self) -> str:
        return self.Config.MetricName

    # ---- saving
    @staticmethod
    def _agreed(opt, metric: float) -> float:
        """The metric as every rank sees it (mean over the ranks under data parallelism): the decision to save must be
        collective, because the optimizer's SaveTo gathers sharded state with a collective call."""
        return float(opt.ReduceMetric(metric)) if opt is not None and hasattr(opt, "ReduceMetric") else float(metric)

    def _write(self, path: str, model, opt, step: int, metric: float, metric_name: str) -> OaStatus:
        primary = opt.IsPrimaryWriter() if opt is not None and hasattr(opt, "IsPrimaryWriter") else True
        if primary:
            os.makedirs(os.path.dirname(path), exist_ok=True)
        oam = OamModel()
        st = model.SaveTo(oam)
        if not st:
            return st
        if opt is not None:
            st = opt.SaveTo(oam)
            if not st:
                return st
        pr = OamProgress()
        pr.Step, pr.BestMetric, pr.LowerIsBetter, pr.MetricName = int(step), float(metric), self.Config.LowerIsBetter, metric_name
        if opt is not None:
            pr.Lr = float(opt.Lr())
        oam.SetProgress(pr)
        return oam.Save(path) if primary else OaStatus.Ok()     # every rank took part in the gather; one rank writes

    def MaybeSave(self, model, opt, step: int, metric: float, force: bool = False, agreed: bool = False) -> OaStatus:
        """Writes the best-model file when the metric improved (or when forced).  `agreed`: the metric is already the
        value every rank holds."""
        if not agreed:
            metric = self._agreed(opt, metric)
        if not (force or self.IsBetter(metric)):
            return OaStatus.Ok()
        if self.Config.SaveBest or force:
            st = self._write(self.GetMasterPath(), model, opt, step, metric, self.Config.MetricName)
            if not st:
                return st
        if self.IsBetter(metric):
            self.BestMetric = float(metric)
        return OaStatus.Ok()

    def SaveIncremental(self, model, opt, step: int, metric: float, metric_name: str = "", agreed: bool = False) -> OaStatus:
        if not agreed:
            metric = self._agreed(opt, metric)
        name = metric_name or self.Config.MetricName
        path = os.path.join(self.GetIncrementalDir(), self.BuildFilename(step, metric, name))
        st = self._write(path, model, opt, step, metric, name)
        if not st:
            return st
        if opt is None or not hasattr(opt, "IsPrimaryWriter") or opt.IsPrimaryWriter():
            self._saved.append((path, float(metric), int(step)))
            self._rotate()
        return OaStatus.Ok()

    def _rotate(self) -> None:
        if self.Config.MaxKeep <= 0:
            return
        self._saved.sort(key=lambda e: -e[2])                     # newest first
        while len(self._saved) > self.Config.MaxKeep:
            path, _, _ = self._saved.pop()
            try:
                os.remove(path)
            except OSError:
                pass

    # ---- loading
    def LoadBestInto(self, model, opt=None) -> OaStatus:
        return model.Load(self.GetMasterPath(), opt)

    def LatestPath(self) -> Optional[str]:
        if self._saved:
            return max(self._saved, key=lambda e: e[2])[0]
        d = self.GetIncrementalDir()
        if not os.path.isdir(d):
            return None
        best, best_step = None, -1
        for f in os.listdir(d):
            m = re.search(r"_step(\d+)_", f)
            if f.endswith(".oam") and m and int(m.group(1)) > best_step:
                best, best_step = os.path.join(d, f), int(m.group(1))
        return best

    def LoadLatestInto(self, model, opt=None) -> OaStatus:
        path = self.LatestPath()
        if path is None:
            return OaStatus.Error(OaStatusCode.NotFound, f"no checkpoint under {self.GetIncrementalDir()}")
        return model.Load(path, opt)
