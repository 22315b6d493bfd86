"""Training configuration records, YAML loading and the memory-budget auto-tuner
(Source/Public/Oa/Ml/Config.h:23-147, Source/Private/Oa/Ml/Budget.cpp)."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional

from ..core.types import OaPrecision


@dataclass
class OaOptimizerConfig:
    Lr: float = 3e-4
    LrMin: float = 1e-5
    Beta1: float = 0.9
    Beta2: float = 0.999
    Epsilon: float = 1e-8
    WeightDecay: float = 0.01
    MaxGradNorm: float = 1.0
    Scheduler: str = "cosine"            # cosine | constant | linear | cosine_restarts
    WarmupSteps: int = 1000
    CycleSteps: int = 0
    CycleMultiplier: float = 1.0

    def MakeScheduler(self, total_steps: int):
        from . import lr_scheduler as S
        if self.Scheduler == "constant":
            return S.OaWarmupScheduler(self.Lr, max(1, self.WarmupSteps)) if self.WarmupSteps > 0 else S.OaCosineScheduler(self.Lr, self.Lr, 1)
        if self.Scheduler == "cosine_restarts":
            return S.OaWarmupScheduler(self.Lr, max(1, self.WarmupSteps), S.OaCosineWarmRestartsScheduler(self.Lr, max(1, self.CycleSteps or total_steps), max(1, int(self.CycleMultiplier)), self.LrMin))
        if self.Scheduler == "linear":
            class _Linear(S.OaLRScheduler):
                def GetLr(s, step, a=self.Lr, b=self.LrMin, n=max(1, total_steps - self.WarmupSteps)):
                    return a + (b - a) * min(1.0, step / n)
            return S.OaWarmupScheduler(self.Lr, max(1, self.WarmupSteps), _Linear())
        return S.OaLinearWarmupCosineScheduler(self.WarmupSteps, total_steps, self.Lr, self.LrMin)


@dataclass
class OaTrainPhaseConfig:
    Id: str = ""
    Steps: int = 0
    Lr: Optional[float] = None
    LrMin: Optional[float] = None
    WarmupSteps: Optional[int] = None
    CheckpointInterval: Optional[int] = None


@dataclass
class OaTrainBaseConfig:
    BatchSize: int = 32
    TotalSteps: int = 100000
    Seed: int = 42
    Precision: OaPrecision = OaPrecision.BF16
    Device: str = "cuda"                 # cuda | cpu
    EvalInterval: int = 1000
    CheckpointInterval: int = 5000
    GradAccumSteps: int = 1
    AugmentationEnabled: bool = False
    NoiseStd: float = 0.0
    Phases: list = field(default_factory=list)

    def UsesPhases(self) -> bool:
        return bool(self.Phases)


_OPT_KEYS = {"lr": "Lr", "lr_min": "LrMin", "beta1": "Beta1", "beta2": "Beta2", "epsilon": "Epsilon", "weight_decay": "WeightDecay",
             "max_grad_norm": "MaxGradNorm", "scheduler": "Scheduler", "warmup_steps": "WarmupSteps", "cycle_steps": "CycleSteps",
             "cycle_multiplier": "CycleMultiplier"}
_TRAIN_KEYS = {"batch_size": "BatchSize", "total_steps": "TotalSteps", "seed": "Seed", "eval_interval": "EvalInterval",
               "checkpoint_interval": "CheckpointInterval", "grad_accum_steps": "GradAccumSteps", "device": "Device"}


def _node(src):
    if isinstance(src, dict):
        return src
    import yaml
    return yaml.safe_load(open(src)) if "\n" not in str(src) and str(src).endswith((".yaml", ".yml")) else yaml.safe_load(src)


def OaLoadOptimizerYaml(src, cfg: Optional[OaOptimizerConfig] = None) -> OaOptimizerConfig:
    cfg = cfg or OaOptimizerConfig()
    for k, attr in _OPT_KEYS.items():
        v = (_node(src) or {}).get("optimizer", {}).get(k)
        if v is not None:
            setattr(cfg, attr, type(getattr(cfg, attr))(v))
    return cfg


def OaLoadTrainBaseYaml(src, cfg: Optional[OaTrainBaseConfig] = None) -> OaTrainBaseConfig:
    cfg = cfg or OaTrainBaseConfig()
    t = (_node(src) or {}).get("training", {})
    for k, attr in _TRAIN_KEYS.items():
        if t.get(k) is not None:
            setattr(cfg, attr, type(getattr(cfg, attr))(t[k]))
    prec = str(t.get("precision", "bf16")).lower()
    cfg.Precision = OaPrecision.FP32 if prec == "fp32" else OaPrecision.BF16
    for ph in t.get("phases", []) or []:
        cfg.Phases.append(OaTrainPhaseConfig(str(ph.get("id", "")), int(ph.get("steps", 0)), ph.get("lr"), ph.get("lr_min"),
                                             ph.get("warmup_steps"), ph.get("checkpoint_interval")))
    return cfg


@dataclass
class OaVRAMBudgetConfig:
    SafetyMarginPercent: float = 0.10
    MinBatchSize: int = 1
    MaxBatchSize: int = 4096
    MinSeqLen: int = 64
    MaxSeqLen: int = 8192
    PreferredBatchSize: int = 0
    PreferredSeqLen: int = 0
    OptimizerStatesPerParam: int = 4     # master + m + v + gradient, in units of BytesPerParam
    BytesPerParam: int = 4


@dataclass
class OaVRAMBudgetResult:
    BatchSize: int = 0
    SeqLen: int = 0
    ModelBytes: int = 0
    ActivationBytes: int = 0
    TotalBytes: int = 0
    AvailableBytes: int = 0
    UtilizationPercent: float = 0.0
    FitsInVRAM: bool = False


def OaComputeVRAMBudget(model_params: int, activation_bytes_per_token: int, cfg: Optional[OaVRAMBudgetConfig] = None,
                        available_bytes: Optional[int] = None) -> OaVRAMBudgetResult:
    """Largest (sequence length, batch) whose model + optimizer + activation bytes fit the device after the safety margin:
    the preferred values when they fit, else the sequence length is halved down to the minimum before the batch is."""
    cfg = cfg or OaVRAMBudgetConfig()
    if available_bytes is None:
        import torch
        available_bytes = torch.cuda.mem_get_info()[1] if torch.cuda.is_available() else 180 * (1 << 30)
    usable = int(available_bytes * (1.0 - cfg.SafetyMarginPercent))
    model = model_params * cfg.BytesPerParam * (1 + cfg.OptimizerStatesPerParam)
    r = OaVRAMBudgetResult(ModelBytes=model, AvailableBytes=available_bytes)
    seq = cfg.PreferredSeqLen or cfg.MaxSeqLen
    batch = cfg.PreferredBatchSize or cfg.MaxBatchSize
    seq, batch = min(max(seq, cfg.MinSeqLen), cfg.MaxSeqLen), min(max(batch, cfg.MinBatchSize), cfg.MaxBatchSize)
    fits = lambda b, s: model + b * s * activation_bytes_per_token <= usable
    while not fits(batch, seq) and batch > cfg.MinBatchSize:
        batch = max(cfg.MinBatchSize, batch // 2)
    while not fits(batch, seq) and seq > cfg.MinSeqLen:
        seq = max(cfg.MinSeqLen, seq // 2)
    r.BatchSize, r.SeqLen = batch, seq
    r.ActivationBytes = batch * seq * activation_bytes_per_token
    r.TotalBytes = model + r.ActivationBytes
    r.FitsInVRAM = r.TotalBytes <= usable
    r.UtilizationPercent = 100.0 * r.TotalBytes / max(1, available_bytes)
    return r


def OaPrintVRAMBudget(r: OaVRAMBudgetResult) -> None:
    gb = 1 << 30
    print(f"memory budget: batch {r.BatchSize} x seq {r.SeqLen}: model+optimizer {r.ModelBytes / gb:.2f} GiB, activations "
          f"{r.ActivationBytes / gb:.2f} GiB, total {r.TotalBytes / gb:.2f} of {r.AvailableBytes / gb:.2f} GiB ({r.UtilizationPercent:.1f} %)"
          f"{'' if r.FitsInVRAM else '  DOES NOT FIT'}")
