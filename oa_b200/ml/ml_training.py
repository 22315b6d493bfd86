"""OaMlTraining: the zero-boilerplate training wrapper (Source/Public/Oa/Ml/Training.h:48-278).  It owns the engine
initialisation, the step iterator, the standard callbacks and the step body, so that a run is
    t = OaMlTraining(model, optimizer, OaMlTrainingConfig(Steps=300, BatchSize=64, SequenceLength=16))
    t.Run(lambda: sampler.Next(), lambda x, y: OaFnLoss.CrossEntropy(model.Forward(x), y.Reshape([y.NumElements()])))
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Optional

from ..core.types import OaPrecision, OaStatus
from ..runtime import engine as RT
from . import autograd as AG
from .callbacks import OaCbCheckpoint, OaCbCsvLogger, OaCbLrScheduler, OaCbProgressBar, OaCbSummary
from .checkpoint import OaCheckpointManager, OaCheckpointManagerConfig
from .training import OaItTraining, OaItTrainingConfig


@dataclass
class OaMlTrainingConfig:
    Steps: int = 100
    BatchSize: int = 1
    SequenceLength: int = 1
    StepsPerEpoch: int = 0
    Precision: OaPrecision = OaPrecision.FP32
    Program: bool = False                 # replay the step as a CUDA graph from step 2 on (static input buffers required)
    ProgressBar: bool = True
    Summary: bool = True
    CsvPath: str = ""
    CheckpointDir: str = ""
    CheckpointEvery: int = 0
    ModelName: str = "OaModule"
    GradAccumSteps: int = 1
    TimerName: str = "train"


class OaMlTraining:
    def __init__(self, model, optimizer, config: Optional[OaMlTrainingConfig] = None, scheduler=None):
        self.Config = config or OaMlTrainingConfig()
        c = self.Config
        if RT.OaEngine.GetGlobal() is None:
            RT.OaInitComputeEngine(RT.OaEngineConfig(Precision=c.Precision))
        self.Model, self.Opt = model, optimizer
        self.Training = OaItTraining(optimizer, OaItTrainingConfig(TotalSteps=c.Steps, BatchSize=c.BatchSize, SequenceLength=c.SequenceLength,
                                                                   StepsPerEpoch=c.StepsPerEpoch, Program=c.Program, TimerName=c.TimerName))
        if c.ProgressBar:
            self.Training.AddCallback(OaCbProgressBar())
        if scheduler is not None:
            self.Training.AddCallback(OaCbLrScheduler(scheduler, optimizer))
        if c.CsvPath:
            self.Training.AddCallback(OaCbCsvLogger(c.CsvPath))
        self.Checkpoints: Optional[OaCheckpointManager] = None
        if c.CheckpointDir:
            self.Checkpoints = OaCheckpointManager(OaCheckpointManagerConfig(Dir=c.CheckpointDir, ModelName=c.ModelName))
            self.Training.AddCallback(OaCbCheckpoint(self.Checkpoints, model, optimizer, c.CheckpointEvery, verbose=False))
        if c.Summary:
            self.Training.AddCallback(OaCbSummary())

    def AddCallback(self, cb) -> None:
        self.Training.AddCallback(cb)

    def Run(self, next_batch: Callable, loss_fn: Callable) -> OaStatus:
        """next_batch() -> (x, y); loss_fn(x, y) -> scalar loss matrix.  With GradAccumSteps = n the optimizer steps once
        per n micro-batches and the loss is scaled by 1 / n so that the accumulated gradient is the mean."""
        from ..core import fn_matrix as F
        tr, n = self.Training, max(1, self.Config.GradAccumSteps)
        while not tr.IsDone():
            self.Opt.ZeroGrad()
            loss = None
            for _ in range(n):
                x, y = next_batch()
                with AG.OaGradientTape() as tape:
                    micro = loss_fn(x, y)
                    scaled = F.Scale(micro, 1.0 / n) if n > 1 else micro
                    tape.Backward(scaled)
                loss = micro
            tr.Next(loss)
        tr.Finish()
        return tr.LastStatus
