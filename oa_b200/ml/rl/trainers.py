"""Actor-critic model, collector, evaluation and the PPO / DQN / SAC trainers.

Reference: Source/Public/Oa/Ml/Rl/{ActorCritic,Collector,Evaluation,ItRlTraining,PpoTrainer,DqnTrainer,SacTrainer}.h and
their implementations under Source/Private/Oa/Ml/Rl/.  Every trainer drives an ordinary OaItTraining for its optimizer
updates, so callbacks, metrics, GPU timing and sessions work as in supervised training.
"""
from __future__ import annotations

import enum
import math
from dataclasses import dataclass, field
from typing import Optional

import torch

from ...core import fn_matrix as F
from ...core.matrix import OaMatrix
from ...core.types import OaStatus, OaStatusCode
from ...runtime import engine as RT
from .. import autograd as AG
from ..module import OaModule
from ..nn.layers import OaLinear
from ..training import OaItTraining, OaItTrainingConfig
from . import fn_rl as FR
from .environment import OaRlEnvironment
from .storage import (OaRlReplayBuffer, OaRlRolloutBatch, OaRlRolloutBuffer, OaRlRolloutConfig, OaRlTransition)


def _err(code, msg):
    return OaStatus.Error(code, msg)


def _prod(shape) -> int:
    n = 1
    for s in shape:
        n *= int(s)
    return n


# ---------------------------------------------------------------------------------------------------- actor / critic
@dataclass
class OaRlActorCriticOutput:
    Logits: Optional[OaMatrix] = None
    Value: Optional[OaMatrix] = None

    def IsValid(self) -> bool:
        return self.Logits is not None and self.Value is not None


class OaRlActorCritic(OaModule):
    """Environment-neutral discrete actor / critic contract: implement Evaluate."""

    def Forward(self, observation: OaMatrix) -> OaMatrix:
        return self.Evaluate(observation).Logits

    def Evaluate(self, observation: OaMatrix) -> OaRlActorCriticOutput:
        raise NotImplementedError


@dataclass
class OaCategoricalActorCriticConfig:
    ObservationSize: int = 0
    ActionCount: int = 0
    HiddenSize: int = 64


class OaCategoricalActorCritic(OaRlActorCritic):
    """Two separate two-hidden-layer ReLU MLPs (children policy.0, policy.1, policy, value.0, value.1, value)."""

    def __init__(self, config: OaCategoricalActorCriticConfig):
        super().__init__()
        self.Config_ = config
        O, Hd, A = config.ObservationSize, config.HiddenSize, config.ActionCount
        self.Policy0 = self.RegisterModule("policy.0", OaLinear(O, Hd))
        self.Policy1 = self.RegisterModule("policy.1", OaLinear(Hd, Hd))
        self.Policy = self.RegisterModule("policy", OaLinear(Hd, A))
        self.Value0 = self.RegisterModule("value.0", OaLinear(O, Hd))
        self.Value1 = self.RegisterModule("value.1", OaLinear(Hd, Hd))
        self.Value = self.RegisterModule("value", OaLinear(Hd, 1))

    @staticmethod
    def Create(config: OaCategoricalActorCriticConfig):
        if config.ObservationSize <= 0 or config.ActionCount <= 1 or config.HiddenSize <= 0:
            return None, _err(OaStatusCode.InvalidArgument, "actor/critic needs positive observation / hidden sizes and at least two actions")
        return OaCategoricalActorCritic(config), OaStatus.Ok()

    def Config(self) -> OaCategoricalActorCriticConfig:
        return self.Config_

    @staticmethod
    def _relu(lin: OaLinear, x: OaMatrix) -> OaMatrix:
        return F.LinearRelu(x, lin.Weight.Data, lin.Bias.Data)

    def Evaluate(self, observation: OaMatrix) -> OaRlActorCriticOutput:
        t = observation.Tensor()
        if t.dtype != torch.float32 or t.dim() != 2 or t.shape[1] != self.Config_.ObservationSize:
            return OaRlActorCriticOutput()
        ph = self._relu(self.Policy1, self._relu(self.Policy0, observation))
        vh = self._relu(self.Value1, self._relu(self.Value0, observation))
        return OaRlActorCriticOutput(self.Policy.Forward(ph), F.Reshape(self.Value.Forward(vh), [t.shape[0]]))


# --------------------------------------------------------------------------------------------- two-phase RL lifecycle
class OaRlTrainingPhase(enum.IntEnum):
    Collect = 0
    Update = 1
    Complete = 2


@dataclass
class OaItRlTrainingConfig:
    Rollouts: int = 0
    Horizon: int = 0
    Environments: int = 0
    UpdateEpochs: int = 0
    TimerName: str = "rl_update"


class OaItRlTraining:
    """Coordinates collect -> update cycles of synchronous on-policy training; each update is one OaItTraining step."""

    def __init__(self, optimizer, config: OaItRlTrainingConfig):
        self.Config_ = config
        ok = config.Rollouts > 0 and config.Horizon > 0 and config.Environments > 0 and config.UpdateEpochs > 0
        self.LastStatus_ = OaStatus.Ok() if ok else _err(OaStatusCode.InvalidArgument, "RL training needs positive rollouts, horizon, environments and update epochs")
        self.Updates_ = OaItTraining(optimizer, OaItTrainingConfig(TotalSteps=max(1, config.Rollouts * config.UpdateEpochs),
                                                                   BatchSize=max(1, config.Horizon * config.Environments),
                                                                   TimerName=config.TimerName))
        self.Phase_ = OaRlTrainingPhase.Collect if ok else OaRlTrainingPhase.Complete
        self.RolloutIndex_ = 0
        self.UpdateEpoch_ = 0
        self._rollout_open = False
        self._body_pending = False

    def BeginRollout(self, rollout: OaRlRolloutBuffer) -> OaStatus:
        if self.Phase_ != OaRlTrainingPhase.Collect or self._rollout_open:
            return _err(OaStatusCode.FailedPrecondition, "a rollout can only begin in the collect phase")
        rollout.Reset()
        self._rollout_open = True
        return OaStatus.Ok()

    def FinalizeRollout(self, rollout: OaRlRolloutBuffer, config: Optional[FR.OaGaeConfig] = None) -> OaStatus:
        if self.Phase_ != OaRlTrainingPhase.Collect or not self._rollout_open:
            return _err(OaStatusCode.FailedPrecondition, "no rollout is open")
        st = rollout.Finalize(config)
        if not st:
            self.LastStatus_ = st
            return st
        self._rollout_open = False
        self.Phase_ = OaRlTrainingPhase.Update
        self.UpdateEpoch_ = 0
        return OaStatus.Ok()

    def BeginUpdate(self) -> bool:
        if self.Phase_ != OaRlTrainingPhase.Update or self._body_pending or not self.LastStatus_:
            return False
        if self.Updates_.IsDone():
            return False
        self._body_pending = True
        return True

    def NextUpdate(self, loss: OaMatrix) -> OaStatus:
        if not self._body_pending:
            return _err(OaStatusCode.FailedPrecondition, "NextUpdate without BeginUpdate")
        self._body_pending = False
        self.Updates_.Next(loss)
        if not self.Updates_.LastStatus:
            self.LastStatus_ = self.Updates_.LastStatus
            return self.LastStatus_
        self.UpdateEpoch_ += 1
        if self.UpdateEpoch_ >= self.Config_.UpdateEpochs:
            self.RolloutIndex_ += 1
            self.Phase_ = OaRlTrainingPhase.Complete if self.RolloutIndex_ >= self.Config_.Rollouts else OaRlTrainingPhase.Collect
        return OaStatus.Ok()

    def Finish(self) -> OaStatus:
        self.Updates_.Finish()
        self.Phase_ = OaRlTrainingPhase.Complete
        return OaStatus.Ok()

    def IsValid(self) -> bool: return bool(self.LastStatus_)
    def IsDone(self) -> bool: return self.Phase_ == OaRlTrainingPhase.Complete or self.Updates_.StopRequested()
    def Phase(self) -> OaRlTrainingPhase: return self.Phase_
    def RolloutIndex(self) -> int: return self.RolloutIndex_
    def UpdateEpoch(self) -> int: return self.UpdateEpoch_
    def Config(self) -> OaItRlTrainingConfig: return self.Config_
    def LastStatus(self) -> OaStatus: return self.LastStatus_
    def UpdateLoop(self) -> OaItTraining: return self.Updates_


# ------------------------------------------------------------------------------------------------------- collector
@dataclass
class OaRlCollectorConfig:
    Horizon: int = 0
    Seed: int = 0
    Gae: FR.OaGaeConfig = field(default_factory=FR.OaGaeConfig)


@dataclass
class OaRlCollectorMetrics:
    Collections: int = 0
    EnvironmentSteps: int = 0
    Transitions: int = 0


class OaRlCollector:
    """Same-device categorical collector: one Collect records a whole rollout (policy, environment step, fused append,
    auto-reset, GAE) on the stream and returns its completion event without waiting."""

    def __init__(self, environment: OaRlEnvironment, model: OaRlActorCritic, config: OaRlCollectorConfig):
        self.Environment_, self.Model_, self.Config_ = environment, model, config
        self.Metrics_ = OaRlCollectorMetrics()
        self.ActionIndex_ = 0

    @staticmethod
    def Create(environment: OaRlEnvironment, model: OaRlActorCritic, config: OaRlCollectorConfig):
        if config.Horizon <= 0:
            return None, _err(OaStatusCode.InvalidArgument, "collector needs a positive horizon")
        return OaRlCollector(environment, model, config), OaStatus.Ok()

    def Metrics(self) -> OaRlCollectorMetrics:
        return self.Metrics_

    def Collect(self, rollout: OaRlRolloutBuffer):
        """Returns (event, status)."""
        env, E = self.Environment_, self.Environment_.Environments()
        if rollout.Capacity() != self.Config_.Horizon or rollout.Config().Environments != E:
            return None, _err(OaStatusCode.InvalidArgument, "rollout shape does not match the collector")
        oe = _prod(env.Spec().Observation.Shape)

        def body() -> OaStatus:
            rollout.Reset()
            with AG.OaGradNo():
                for _ in range(self.Config_.Horizon):
                    obs = OaMatrix(env.Observation().Tensor().clone())
                    net = self.Model_.Evaluate(F.Reshape(obs, [E, oe]))
                    if not net.IsValid():
                        return _err(OaStatusCode.FailedPrecondition, "actor/critic evaluation failed")
                    self.ActionIndex_ += 1
                    pol = FR.SampleCategoricalPolicy(net.Logits, net.Value, self.Config_.Seed + self.ActionIndex_)
                    if not pol.IsValid():
                        return _err(OaStatusCode.FailedPrecondition, "policy sampling failed")
                    tr, st = env.StepEnvironment(pol.Action)
                    if not st:
                        return st
                    nxt = self.Model_.Evaluate(F.Reshape(tr.NextObservation, [E, oe]))
                    st = rollout.Append(OaRlTransition(tr.Observation, pol.Action, tr.Reward, pol.Value, nxt.Value, pol.LogProbability,
                                                       tr.Terminated, tr.Truncated))
                    if not st:
                        return st
                    st = env.ResetCompleted()
                    if not st:
                        return st
            return rollout.Finalize(self.Config_.Gae)

        st = env.RecordCommands(body)
        if not st:
            return None, st
        ev, st = env.Submit()
        if st:
            self.Metrics_.Collections += 1
            self.Metrics_.EnvironmentSteps += self.Config_.Horizon
            self.Metrics_.Transitions += self.Config_.Horizon * E
        return ev, st


# ------------------------------------------------------------------------------------------------------ evaluation
@dataclass
class OaRlEvaluationConfig:
    Horizon: int = 1000
    Seed: int = 1


@dataclass
class OaRlEvaluationMetrics:
    EnvironmentSteps: int = 0
    Transitions: int = 0
    CompletedEpisodes: int = 0
    MeanCompletedReturn: float = 0.0
    MinimumCompletedReturn: float = 0.0
    MaximumCompletedReturn: float = 0.0


def EvaluateCategorical(environment: OaRlEnvironment, model: OaRlActorCritic, config: Optional[OaRlEvaluationConfig] = None):
    """Greedy evaluation over `Horizon` vector steps: the whole horizon is launched first, then one synchronisation and
    three compact readbacks (reward, terminated, truncated).  Returns (metrics, status)."""
    cfg = config or OaRlEvaluationConfig()
    E = environment.Environments()
    if cfg.Horizon <= 0:
        return None, _err(OaStatusCode.InvalidArgument, "evaluation needs a positive horizon")
    oe = _prod(environment.Spec().Observation.Shape)
    rollout, st = OaRlRolloutBuffer.Create(OaRlRolloutConfig(cfg.Horizon, E, tuple(environment.Spec().Observation.Shape)))
    if not st:
        return None, st

    def body() -> OaStatus:
        rollout.Reset()
        st = environment.ResetEnvironment(cfg.Seed)
        if not st:
            return st
        with AG.OaGradNo():
            for _ in range(cfg.Horizon):
                net = model.Evaluate(F.Reshape(OaMatrix(environment.Observation().Tensor().clone()), [E, oe]))
                if not net.IsValid():
                    return _err(OaStatusCode.FailedPrecondition, "actor/critic evaluation failed")
                action = FR.SampleLogits(net.Logits, 0.0, 0, 1.0, cfg.Seed)
                pol = FR.EvaluateCategoricalPolicy(net.Logits, action, net.Value)
                tr, st = environment.StepEnvironment(action)
                if not st:
                    return st
                st = rollout.Append(OaRlTransition(tr.Observation, action, tr.Reward, net.Value, net.Value, pol.LogProbability,
                                                   tr.Terminated, tr.Truncated))
                if not st:
                    return st
                st = environment.ResetCompleted()
                if not st:
                    return st
        return OaStatus.Ok()

    st = environment.RecordCommands(body)
    if not st:
        return None, st
    ev, st = environment.Submit()
    if not st:
        return None, st
    st = environment.Wait(ev)
    if not st:
        return None, st
    B = rollout.Batch()
    reward = B.Reward.Tensor().cpu()
    ended = (B.Terminated.Tensor().cpu().ne(0) | B.Truncated.Tensor().cpu().ne(0))
    run = torch.zeros(E)
    finished = []
    for t in range(cfg.Horizon):
        run += reward[t]
        idx = ended[t].nonzero().flatten()
        if idx.numel():
            finished.extend(run[idx].tolist())
            run[idx] = 0.0
    m = OaRlEvaluationMetrics(EnvironmentSteps=cfg.Horizon, Transitions=cfg.Horizon * E, CompletedEpisodes=len(finished))
    if finished:
        m.MeanCompletedReturn = sum(finished) / len(finished)
        m.MinimumCompletedReturn, m.MaximumCompletedReturn = min(finished), max(finished)
    return m, OaStatus.Ok()


# -------------------------------------------------------------------------------------------------------------- PPO
@dataclass
class OaPpoTrainerConfig:
    Rollouts: int = 0
    Horizon: int = 0
    Environments: int = 0
    UpdateEpochs: int = 0
    ObservationShape: tuple = ()
    Seed: int = 0
    Gae: FR.OaGaeConfig = field(default_factory=FR.OaGaeConfig)
    Loss: FR.OaPpoLossConfig = field(default_factory=FR.OaPpoLossConfig)


@dataclass
class OaPpoTrainerMetrics:
    Rollout: int = 0
    UpdateEpoch: int = 0
    TotalLoss: float = 0.0
    PolicyLoss: float = 0.0
    ValueLoss: float = 0.0
    Entropy: float = 0.0


class OaPpoTrainer:
    """Complete categorical PPO loop; the environment stays with the caller.  Cycle: BeginCollection, Horizon x
    (Act, environment step, Observe), EndCollection (GAE), UpdateEpochs x Update."""

    def __init__(self, model: OaRlActorCritic, optimizer, config: OaPpoTrainerConfig, rollout: OaRlRolloutBuffer):
        self.Model, self.Optimizer, self.Config_, self.Rollout = model, optimizer, config, rollout
        self.Training = OaItRlTraining(optimizer, OaItRlTrainingConfig(config.Rollouts, config.Horizon, config.Environments,
                                                                       config.UpdateEpochs, "ppo_update"))
        self.Metrics_ = OaPpoTrainerMetrics()
        self.Collecting = False
        self.ActionIndex = 0

    @staticmethod
    def Create(model: OaRlActorCritic, optimizer, config: OaPpoTrainerConfig):
        if min(config.Rollouts, config.Horizon, config.Environments, config.UpdateEpochs) <= 0 or not config.ObservationShape:
            return None, _err(OaStatusCode.InvalidArgument, "PPO needs positive rollouts, horizon, environments, update epochs and an observation shape")
        rollout, st = OaRlRolloutBuffer.Create(OaRlRolloutConfig(config.Horizon, config.Environments, tuple(config.ObservationShape)))
        if not st:
            return None, st
        t = OaPpoTrainer(model, optimizer, config, rollout)
        return (t, OaStatus.Ok()) if t.Training.IsValid() else (None, t.Training.LastStatus())

    def BeginCollection(self) -> OaStatus:
        if self.Collecting or self.Training.Phase() != OaRlTrainingPhase.Collect:
            return _err(OaStatusCode.FailedPrecondition, "collection cannot begin in the current phase")
        st = self.Training.BeginRollout(self.Rollout)
        self.Collecting = bool(st)
        return st

    def _flat(self, obs: OaMatrix) -> OaMatrix:
        return F.Reshape(obs, [self.Config_.Environments, _prod(self.Config_.ObservationShape)])

    def Act(self, observation: OaMatrix) -> FR.OaRlPolicyResult:
        if not self.Collecting:
            return FR.OaRlPolicyResult()
        with AG.OaGradNo():
            net = self.Model.Evaluate(self._flat(observation))
            if not net.IsValid():
                return FR.OaRlPolicyResult()
            self.ActionIndex += 1
            return FR.SampleCategoricalPolicy(net.Logits, net.Value, self.Config_.Seed + self.ActionIndex)

    def Observe(self, observation, next_observation, reward, terminated, truncated, policy: FR.OaRlPolicyResult) -> OaStatus:
        if not self.Collecting or not policy.IsValid():
            return _err(OaStatusCode.FailedPrecondition, "Observe requires active collection and a valid policy result")
        with AG.OaGradNo():
            nxt = self.Model.Evaluate(self._flat(next_observation))
        if not nxt.IsValid():
            return _err(OaStatusCode.FailedPrecondition, "next-value evaluation failed")
        return self.Rollout.Append(OaRlTransition(observation, policy.Action, reward, policy.Value, nxt.Value, policy.LogProbability,
                                                  terminated, truncated))

    def EndCollection(self) -> OaStatus:
        if not self.Collecting:
            return _err(OaStatusCode.FailedPrecondition, "collection is not active")
        st = self.Training.FinalizeRollout(self.Rollout, self.Config_.Gae)
        if st:
            self.Collecting = False
        return st

    def Update(self) -> OaStatus:
        """One PPO epoch over the whole rollout.  Call until NeedsCollection() or IsDone()."""
        if self.Training.Phase() != OaRlTrainingPhase.Update:
            return _err(OaStatusCode.FailedPrecondition, "cannot update in the current phase")
        if not self.Training.BeginUpdate():
            if self.Training.UpdateLoop().StopRequested():
                return self.Training.Finish()
            return self.Training.LastStatus() if not self.Training.LastStatus() else _err(OaStatusCode.FailedPrecondition, "update did not begin")
        cfg, B = self.Config_, self.Rollout.Batch()
        n = cfg.Environments * cfg.Horizon
        obs = F.Reshape(B.Observation, [n, _prod(cfg.ObservationShape)])
        flat = lambda m: F.Reshape(m, [n])
        self.Optimizer.ZeroGrad()
        tape = AG.OaGradientTape()
        net = self.Model.Evaluate(obs)
        pol = FR.EvaluateCategoricalPolicy(net.Logits, flat(B.Action), net.Value) if net.IsValid() else FR.OaRlPolicyResult()
        if not pol.IsValid():
            return _err(OaStatusCode.FailedPrecondition, "action re-evaluation failed")
        adv = FR.NormalizeAdvantages(flat(B.Advantage))
        loss = FR.Ppo(pol.LogProbability, flat(B.OldLogProbability), adv, pol.Value, flat(B.Return), pol.Entropy, cfg.Loss)
        if not loss.IsValid():
            return _err(OaStatusCode.FailedPrecondition, "loss construction failed")
        tape.Backward(loss.TotalLoss)
        tape.Close()
        st = self.Training.NextUpdate(loss.TotalLoss)
        if not st:
            return st
        self.Metrics_ = OaPpoTrainerMetrics(self.Training.RolloutIndex(), self.Training.UpdateEpoch(), self.Training.UpdateLoop().LastLoss(),
                                            loss.PolicyLoss.Item(), loss.ValueLoss.Item(), loss.Entropy.Item())
        if self.Training.IsDone():
            return self.Training.Finish()
        return OaStatus.Ok()

    def IsValid(self) -> bool: return self.Training.IsValid()
    def IsDone(self) -> bool: return self.Training.IsDone()
    def NeedsCollection(self) -> bool: return not self.Collecting and self.Training.Phase() == OaRlTrainingPhase.Collect
    def Phase(self) -> OaRlTrainingPhase: return self.Training.Phase()
    def Config(self) -> OaPpoTrainerConfig: return self.Config_
    def Metrics(self) -> OaPpoTrainerMetrics: return self.Metrics_
    def Batch(self) -> OaRlRolloutBatch: return self.Rollout.Batch()
    def TrainingLoop(self) -> OaItTraining: return self.Training.UpdateLoop()
    def Save(self, path) -> OaStatus: return self.Model.Save(path, self.Optimizer)
    def Load(self, path) -> OaStatus: return self.Model.Load(path, self.Optimizer)


# ---------------------------------------------------------------------------------------------------------- DQN / SAC
def CopyModel(source: OaModule, target: OaModule) -> OaStatus:
    """Hard parameter copy between two modules of identical structure (target-network synchronisation)."""
    src, dst = source.AllNamedParameterPtrs(), target.AllNamedParameterPtrs()
    if len(src) != len(dst):
        return _err(OaStatusCode.InvalidArgument, "target network has a different parameter count")
    for a, b in zip(src, dst):
        ta, tb = a.Param.Data.Tensor(), b.Param.Data.Tensor()
        if ta.shape != tb.shape or ta.dtype != tb.dtype:
            return _err(OaStatusCode.InvalidArgument, f"target parameter {b.Name} does not match {a.Name}")
    F._ctx_add("CopyModel")
    with torch.no_grad():
        for a, b in zip(src, dst):
            b.Param.Data.Tensor().copy_(a.Param.Data.Tensor())
    return OaStatus.Ok()


@dataclass
class OaDqnTrainerConfig:
    Updates: int = 0
    BatchSize: int = 0
    TargetUpdateInterval: int = 100
    ObservationShape: tuple = ()
    Seed: int = 0
    Loss: FR.OaDqnLossConfig = field(default_factory=FR.OaDqnLossConfig)


@dataclass
class OaDqnTrainerMetrics:
    Update: int = 0
    Loss: float = 0.0


class OaDqnTrainer:
    def __init__(self, online, target, optimizer, replay: OaRlReplayBuffer, config: OaDqnTrainerConfig):
        self.Online, self.Target, self.Optimizer, self.Replay, self.Config_ = online, target, optimizer, replay, config
        self.Training = OaItTraining(optimizer, OaItTrainingConfig(TotalSteps=config.Updates, BatchSize=config.BatchSize, TimerName="dqn_update"))
        self.Metrics_ = OaDqnTrainerMetrics()

    @staticmethod
    def Create(online: OaModule, target: OaModule, optimizer, replay: OaRlReplayBuffer, config: OaDqnTrainerConfig):
        rc = replay.Config()
        if (config.Updates <= 0 or config.BatchSize <= 0 or config.TargetUpdateInterval <= 0 or tuple(config.ObservationShape) != tuple(rc.ObservationShape)
                or rc.ActionShape or rc.ActionDtype.name != "Int32"):
            return None, _err(OaStatusCode.InvalidArgument, "DQN configuration does not match discrete replay storage")
        st = CopyModel(online, target)
        if not st:
            return None, st
        return OaDqnTrainer(online, target, optimizer, replay, config), OaStatus.Ok()

    def Update(self) -> OaStatus:
        tr = self.Training
        if tr.StopRequested():
            tr.Finish()
            return OaStatus.Ok()
        if self.IsDone():
            return OaStatus.Ok()
        cfg = self.Config_
        if self.Replay.Size() < cfg.BatchSize:
            return _err(OaStatusCode.FailedPrecondition, "replay does not contain one complete batch")
        if tr.IsDone():
            return OaStatus.Ok()
        batch, st = self.Replay.Sample(cfg.BatchSize, cfg.Seed + self.Metrics_.Update + 1)
        if not st:
            return st
        oe = _prod(cfg.ObservationShape)
        obs, nxt = F.Reshape(batch.Observation, [cfg.BatchSize, oe]), F.Reshape(batch.NextObservation, [cfg.BatchSize, oe])
        with AG.OaGradNo():
            next_q = self.Target.Forward(nxt)
        self.Optimizer.ZeroGrad()
        tape = AG.OaGradientTape()
        q = self.Online.Forward(obs)
        loss = FR.Dqn(q, batch.Action, batch.Reward, next_q, batch.Terminated, batch.Truncated, cfg.Loss)
        if not loss.IsValid():
            return _err(OaStatusCode.FailedPrecondition, "loss construction failed")
        tape.Backward(loss.Loss)
        tape.Close()
        tr.Next(loss.Loss)
        if not tr.LastStatus:
            return tr.LastStatus
        self.Metrics_ = OaDqnTrainerMetrics(tr.Index(), tr.LastLoss())
        if self.Metrics_.Update % cfg.TargetUpdateInterval == 0:
            st = self.SyncTarget()
            if not st:
                return st
        if tr.StepCount() >= tr.TotalSteps():
            tr.Finish()
        return OaStatus.Ok()

    def SyncTarget(self) -> OaStatus:
        return CopyModel(self.Online, self.Target)

    def IsDone(self) -> bool: return self.Training.StopRequested() or self.Training.StepCount() >= self.Training.TotalSteps()
    def Metrics(self) -> OaDqnTrainerMetrics: return self.Metrics_
    def TrainingLoop(self) -> OaItTraining: return self.Training
    def Save(self, path) -> OaStatus: return self.Online.Save(path, self.Optimizer)

    def Load(self, path) -> OaStatus:
        st = self.Online.Load(path, self.Optimizer)
        return self.SyncTarget() if st else st


@dataclass
class OaSacTrainerConfig:
    Updates: int = 0
    BatchSize: int = 0
    ActionDimensions: int = 0
    TargetUpdateInterval: int = 1
    ObservationShape: tuple = ()
    ActionMinimum: float = -1.0
    ActionMaximum: float = 1.0
    Seed: int = 0
    Loss: FR.OaSacLossConfig = field(default_factory=FR.OaSacLossConfig)


@dataclass
class OaSacTrainerMetrics:
    Update: int = 0
    ActorLoss: float = 0.0
    CriticLoss: float = 0.0


class OaSacTrainer:
    """Fixed-alpha soft actor-critic.  The actor's Forward returns [B, 2A] (mean then log-std); each critic takes
    [observation, action] concatenated on the last axis and returns [B] or [B, 1].  Two optimizer units per update:
    the critic loop is the primary controller, the actor loop is observable separately."""

    def __init__(self, actor, c1, c2, t1, t2, actor_opt, critic_opt, replay, config: OaSacTrainerConfig):
        self.Actor, self.Critic1, self.Critic2, self.Target1, self.Target2 = actor, c1, c2, t1, t2
        self.ActorOpt, self.CriticOpt, self.Replay, self.Config_ = actor_opt, critic_opt, replay, config
        mk = lambda opt, name: OaItTraining(opt, OaItTrainingConfig(TotalSteps=config.Updates, BatchSize=config.BatchSize, TimerName=name))
        self.CriticTraining, self.ActorTraining = mk(critic_opt, "sac_critic_update"), mk(actor_opt, "sac_actor_update")
        self.Metrics_ = OaSacTrainerMetrics()

    @staticmethod
    def Create(actor, critic1, critic2, target1, target2, actor_opt, critic_opt, replay: OaRlReplayBuffer, config: OaSacTrainerConfig):
        rc = replay.Config()
        ok = (config.Updates > 0 and config.BatchSize > 0 and config.ActionDimensions > 0 and config.TargetUpdateInterval > 0
              and tuple(config.ObservationShape) == tuple(rc.ObservationShape) and rc.ActionDtype.name == "Float32"
              and tuple(rc.ActionShape) == (config.ActionDimensions,) and math.isfinite(config.ActionMinimum)
              and math.isfinite(config.ActionMaximum) and config.ActionMinimum < config.ActionMaximum)
        if not ok:
            return None, _err(OaStatusCode.InvalidArgument, "SAC configuration does not match continuous replay storage")
        for s, t in ((critic1, target1), (critic2, target2)):
            st = CopyModel(s, t)
            if not st:
                return None, st
        return OaSacTrainer(actor, critic1, critic2, target1, target2, actor_opt, critic_opt, replay, config), OaStatus.Ok()

    def _policy(self, obs: OaMatrix, seed: int) -> FR.OaRlContinuousPolicyResult:
        cfg = self.Config_
        out = self.Actor.Forward(obs)
        if out.Tensor().dim() != 2 or out.Tensor().shape[1] != 2 * cfg.ActionDimensions:
            return FR.OaRlContinuousPolicyResult()
        mean, log_std = F.Split(out, [cfg.ActionDimensions, cfg.ActionDimensions], -1)
        value = F.Zeros([cfg.BatchSize], dtype=torch.float32)
        return FR.SampleTanhNormalPolicy(mean, log_std, value, cfg.ActionMinimum, cfg.ActionMaximum, seed)

    def _q(self, critic, obs, action) -> Optional[OaMatrix]:
        q = critic.Forward(F.Concat([obs, action], -1))
        t = q.Tensor()
        B = self.Config_.BatchSize
        if tuple(t.shape) == (B,):
            return q
        return F.Reshape(q, [B]) if tuple(t.shape) == (B, 1) else None

    def Update(self) -> OaStatus:
        cfg, ct, at = self.Config_, self.CriticTraining, self.ActorTraining
        if ct.StopRequested():
            ct.Finish()
            at.RequestStop()
            at.Finish()
            return OaStatus.Ok()
        if self.IsDone():
            return OaStatus.Ok()
        if self.Replay.Size() < cfg.BatchSize:
            return _err(OaStatusCode.FailedPrecondition, "replay does not contain one complete batch")
        if ct.IsDone():
            return OaStatus.Ok()
        batch, st = self.Replay.Sample(cfg.BatchSize, cfg.Seed + self.Metrics_.Update + 1)
        if not st:
            return st
        B, oe = cfg.BatchSize, _prod(cfg.ObservationShape)
        obs, nxt = F.Reshape(batch.Observation, [B, oe]), F.Reshape(batch.NextObservation, [B, oe])
        stored_action = F.Reshape(batch.Action, [B, cfg.ActionDimensions])
        with AG.OaGradNo():
            next_pol = self._policy(nxt, cfg.Seed + 0x100000001 + self.Metrics_.Update)
            if not next_pol.IsValid():
                return _err(OaStatusCode.InvalidArgument, "actor must return [B, 2 * action-dim]")
            nq1, nq2 = self._q(self.Target1, nxt, next_pol.Action), self._q(self.Target2, nxt, next_pol.Action)
        if nq1 is None or nq2 is None:
            return _err(OaStatusCode.InvalidArgument, "critics must return [B] or [B, 1]")
        # ---- critic unit
        self.CriticOpt.ZeroGrad()
        tape = AG.OaGradientTape()
        q1, q2 = self._q(self.Critic1, obs, stored_action), self._q(self.Critic2, obs, stored_action)
        closs = FR.SacCritic(q1, q2, batch.Reward, nq1, nq2, next_pol.LogProbability, batch.Terminated, batch.Truncated, cfg.Loss)
        if not closs.IsValid():
            return _err(OaStatusCode.FailedPrecondition, "critic loss failed")
        tape.Backward(closs.TotalLoss)
        tape.Close()
        ct.Next(closs.TotalLoss)
        if not ct.LastStatus:
            return ct.LastStatus
        self.Metrics_.CriticLoss = ct.LastLoss()
        # ---- actor unit (critic gradients produced here are discarded by the next ZeroGrad)
        if at.IsDone():
            return _err(OaStatusCode.FailedPrecondition, "actor iterator completed before the critic iterator")
        self.ActorOpt.ZeroGrad()
        self.CriticOpt.ZeroGrad()
        tape = AG.OaGradientTape()
        pol = self._policy(obs, cfg.Seed + 0x200000001 + self.Metrics_.Update)
        if not pol.IsValid():
            return _err(OaStatusCode.FailedPrecondition, "actor policy failed")
        aq1, aq2 = self._q(self.Critic1, obs, pol.Action), self._q(self.Critic2, obs, pol.Action)
        aloss = FR.SacActor(aq1, aq2, pol.LogProbability, cfg.Loss.EntropyCoefficient)
        if aloss is None:
            return _err(OaStatusCode.FailedPrecondition, "actor loss failed")
        tape.Backward(aloss)
        tape.Close()
        at.Next(aloss)
        if not at.LastStatus:
            return at.LastStatus
        self.Metrics_.ActorLoss = at.LastLoss()
        self.Metrics_.Update = ct.StepCount()
        if self.Metrics_.Update % cfg.TargetUpdateInterval == 0:
            st = self.SyncTargets()
            if not st:
                return st
        if self.Metrics_.Update >= cfg.Updates:
            ct.Finish()
            at.Finish()
        return OaStatus.Ok()

    def SyncTargets(self) -> OaStatus:
        st = CopyModel(self.Critic1, self.Target1)
        return CopyModel(self.Critic2, self.Target2) if st else st

    def IsDone(self) -> bool: return self.CriticTraining.StopRequested() or self.CriticTraining.StepCount() >= self.CriticTraining.TotalSteps()
    def Metrics(self) -> OaSacTrainerMetrics: return self.Metrics_
    def TrainingLoop(self) -> OaItTraining: return self.CriticTraining
    def ActorTrainingLoop(self) -> OaItTraining: return self.ActorTraining
